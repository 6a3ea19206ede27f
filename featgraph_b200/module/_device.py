"""Device plumbing shared by the SpMM / SDDMM modules: torch owns device memory and
streams, the C ABI does the work."""
import ctypes

import numpy as np
import torch

from .. import _native


def resolve_device(device=None):
    """The reference pins everything to ``tvm.gpu(0)`` (python/featgraph/module/spmm.py:218);
    here the default is the current CUDA device.  No CUDA device -> RuntimeError: there is
    no CPU execution path in this library."""
    if not torch.cuda.is_available():
        raise RuntimeError(
            "featgraph_b200 needs a CUDA device (sm_100a): the SpMM/SDDMM kernels have no CPU fallback")
    if device is None:
        return torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)
    if device.type != "cuda":
        raise RuntimeError("featgraph_b200 runs on CUDA devices only, got %s" % (device,))
    if device.index is None:
        device = torch.device("cuda", torch.cuda.current_device())
    return device


def upload(array, device, dtype=None):
    """One-off copy of a host index/value array to the device (contiguous)."""
    a = np.ascontiguousarray(array, dtype=dtype)
    return torch.from_numpy(a).to(device)


def ptr(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() > 0 else ctypes.c_void_p(0)


def stream_ptr(device):
    return ctypes.c_void_p(torch.cuda.current_stream(device).cuda_stream)


def check_input(t, shape, device, what):
    if not isinstance(t, torch.Tensor):
        raise TypeError("%s: expected a torch.Tensor on %s, got %r" % (what, device, type(t)))
    if t.device != device:
        raise ValueError("%s lives on %s, the module on %s" % (what, t.device, device))
    if t.dtype != torch.float32:
        raise TypeError("%s must be float32, got %s" % (what, t.dtype))
    if tuple(t.shape) != tuple(shape):
        raise ValueError("%s has shape %s, built for %s" % (what, tuple(t.shape), tuple(shape)))
    if not t.is_contiguous():
        raise ValueError("%s must be contiguous (row-major)" % (what,))
    return t


class _DeviceInt32View:
    """Exposes library-owned device memory through __cuda_array_interface__."""

    def __init__(self, address, count):
        self.__cuda_array_interface__ = {
            "shape": (int(count),), "typestr": "<i4", "data": (int(address), False), "version": 2}


def view_device_int32(address, count, device):
    """Torch view (treat as read-only) of ``count`` int32 at a device address owned by the library."""
    return torch.as_tensor(_DeviceInt32View(address, count), device=device)


def time_calls(fn, device, num_runs):
    """Mean seconds of ``num_runs`` back-to-back calls after one untimed warm-up call, the
    protocol of the reference's timer (python/featgraph/module/spmm.py:179-185: time_evaluator
    with number=num_runs, repeat=1)."""
    num_runs = int(num_runs)
    assert num_runs >= 1
    with torch.cuda.device(device):
        stream = torch.cuda.current_stream(device)
        fn()
        stream.synchronize()
        start = torch.cuda.Event(enable_timing=True)
        stop = torch.cuda.Event(enable_timing=True)
        start.record(stream)
        for _ in range(num_runs):
            fn()
        stop.record(stream)
        stop.synchronize()
        return start.elapsed_time(stop) * 1e-3 / num_runs


# Deferred host-buffer calls (run_host(wait=False)) leave a module's staging buffers in use until the
# next host_sync() on that device; a module that is called again before that would overwrite them
# under a kernel that still reads them.  Each host_sync() starts a new epoch per device; a module
# remembers the epoch of its pending deferred call and refuses further calls within it.
_sync_epoch = {}


def sync_epoch(device):
    return _sync_epoch.get(device.index, 0)


def note_host_sync(device):
    _sync_epoch[device.index] = _sync_epoch.get(device.index, 0) + 1


def refuse_if_deferred_pending(module):
    if getattr(module, "_deferred_epoch", None) == sync_epoch(module._device):
        raise RuntimeError("this module has a deferred run_host(wait=False) call in flight: call "
                           "featgraph_b200.host_sync() before using the module again (its staging "
                           "buffers are still being read)")


lib = _native.lib
check = _native.check
