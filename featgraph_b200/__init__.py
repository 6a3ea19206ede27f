"""featgraph_b200: vanilla SpMM / SDDMM for NVIDIA B200 (sm_100a) behind the module
interface of dglai/FeatGraph (``featgraph.module``, ``featgraph.util``)."""
from . import util
from .placeholder import Placeholder, placeholder

__all__ = ["util", "module", "placeholder", "Placeholder"]


def __getattr__(name):
    # the module layer needs torch; import it on first use so that the host-side
    # utilities stay importable on their own
    if name in ("module", "op", "graphgen", "sharded", "graph_capture"):
        import importlib
        return importlib.import_module("." + name, __name__)
    raise AttributeError(name)


def host_sync(device=None):
    """Wait for every ``run_host(..., wait=False)`` call issued by this thread."""
    import ctypes
    import torch
    from . import _native
    from .module import _device
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    with torch.cuda.device(dev):
        _native.check(_native.lib().fg_host_sync(ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream)))
    _device.note_host_sync(dev)  # modules with a deferred call pending on this device are usable again
