"""SpMM modules: same lifecycle and names as python/featgraph/module/spmm.py of the
reference (construct from a scipy adjacency, ``build``, ``run``, ``measure_average_time``),
executed by hand-written sm_100a kernels through the C ABI instead of generated code.

Both classes run on the GPU.  ``VanillaSpMMx86`` keeps the x86 class's knobs and its
summation order (with ``num_col_partitions`` > 1 that is the DDS order: per column
partition partial sums added in partition order, python/featgraph/op/vanilla_spmm.py:195-218);
``VanillaSpMMcuda`` is plain CSR.  ``target`` keeps the reference's labels ('llvm' / 'cuda').
"""
import ctypes

import numpy as np
import torch

from ..placeholder import check_float32, static_shape
from ..util import util_convert_csr_to_dds
from . import _device as dev


class SpMMbase:
    """Counterpart of ``SpMMbase`` (python/featgraph/module/spmm.py:12-194)."""

    _compute_keys = ()
    _schedule_keys = ()

    def __init__(self, adj_scipy, num_col_partitions=1, device=None, long_row_threshold=0):
        # CSR in SpMM-like kernels (reference :26-29)
        adj_csr = adj_scipy.tocsr() if adj_scipy.format != "csr" else adj_scipy
        self._num_rows, self._num_cols = adj_csr.shape
        assert num_col_partitions >= 1, "num_col_partitions should be larger than or equal to 1"
        self._num_col_partitions = int(num_col_partitions)
        self._target = None
        self._register()
        self._device = dev.resolve_device(device)
        self._nnz = int(adj_csr.indices.shape[0])
        if adj_csr.indptr.dtype != np.int32 or adj_csr.indices.dtype != np.int32:
            raise TypeError("int32 CSR index arrays are required (got %s / %s)"
                            % (adj_csr.indptr.dtype, adj_csr.indices.dtype))
        if adj_csr.data.dtype != np.float32:
            raise TypeError("float32 adjacency values are required, got %s" % adj_csr.data.dtype)

        # an unweighted adjacency (all values exactly 1.0) needs no value array on the device
        unit_values = bool(self._nnz == 0 or np.all(adj_csr.data == np.float32(1.0)))
        self._unit_values = unit_values
        L = dev.lib()
        with torch.cuda.device(self._device):
            indptr = dev.upload(adj_csr.indptr, self._device)
            indices = dev.upload(adj_csr.indices, self._device)
            dev.check(L.fg_csr_validate(dev.ptr(indptr), dev.ptr(indices), self._num_rows,
                                        self._num_cols, self._nnz, dev.stream_ptr(self._device)))
            # heavy-rows-first visiting order, shared by the CSR and DDS kernels
            self._schedule = ctypes.c_void_p()
            dev.check(L.fg_row_schedule_create(dev.ptr(indptr), self._num_rows,
                                               int(long_row_threshold),
                                               dev.stream_ptr(self._device),
                                               ctypes.byref(self._schedule)))
            if self._num_col_partitions > 1:
                # 1-D column partitioning -> DDS arrays (reference :41-56)
                s1_pos, s1_idx, vals = util_convert_csr_to_dds(adj_csr, self._num_col_partitions)
                self._adj_pos = dev.upload(s1_pos, self._device)
                self._adj_idx = dev.upload(s1_idx, self._device)
                self._adj_vals = None if unit_values else dev.upload(vals, self._device)
            else:
                self._adj_pos = indptr
                self._adj_idx = indices
                self._adj_vals = None if unit_values else dev.upload(adj_csr.data, self._device)
        self._feat_shape = None
        self._feat_tile = 0
        self._x_staging = None
        self.out = None

    def __del__(self):
        sched = getattr(self, "_schedule", None)
        if sched is not None and sched.value:
            try:
                dev.lib().fg_row_schedule_destroy(sched)
            except Exception:
                pass
            self._schedule = None

    def _register(self):
        raise NotImplementedError("Please register target.")

    # -- build --------------------------------------------------------------------------
    def _plan(self, input_placeholders, compute_args, schedule_args):
        compute_args = dict(compute_args or {})
        schedule_args = dict(schedule_args or {})
        for k in compute_args:
            if k not in self._compute_keys:
                raise TypeError("unexpected compute argument %r" % (k,))
        for k in schedule_args:
            if k not in self._schedule_keys:
                raise TypeError("unexpected schedule argument %r" % (k,))
        if len(input_placeholders) != 1:
            raise TypeError("SpMM takes one input (the source feature matrix)")
        shape = static_shape(input_placeholders[0])
        check_float32(input_placeholders[0])
        if len(shape) != 2 or shape[0] != self._num_cols:
            raise ValueError("feature matrix must be [num_cols=%d, feat_len], got %s"
                             % (self._num_cols, shape))
        d = shape[1]
        nfp = int(compute_args.get("num_feat_partitions", 1))
        if nfp < 1 or d % nfp != 0:
            raise ValueError("feat_len %d is not divisible by num_feat_partitions %d" % (d, nfp))
        tile = int(schedule_args.get("feat_tile", 0))
        if tile == 0 and nfp > 1:
            # the reference's feature tiling knob doubles as the L2 tile width when it is usable
            f = d // nfp
            if 4 <= f <= 128 and (f & (f - 1)) == 0:
                tile = f
        return shape, d, nfp, tile

    def build(self, input_placeholders, compute_args, schedule_args):
        """Fix the feature shape and allocate the (reused) output
        (reference :81-111; ``out`` plays the role of ``out_tvm``)."""
        shape, d, _, tile = self._plan(input_placeholders, compute_args, schedule_args)
        self._feat_shape = shape
        self._feat_tile = tile
        self.out = torch.zeros((self._num_rows, d), dtype=torch.float32, device=self._device)

    def lower_to_ir(self, input_placeholders, compute_args, schedule_args):
        """Text description of what ``build`` + ``run`` would launch (the reference returns
        the lowered loop nest for debugging, :113-140)."""
        shape, d, nfp, tile = self._plan(input_placeholders, compute_args, schedule_args)
        layout = ("dds(num_col_partitions=%d)" % self._num_col_partitions
                  if self._num_col_partitions > 1 else "csr")
        return ("featgraph_b200 spmm: layout=%s rows=%d cols=%d nnz=%d feat_len=%d "
                "num_feat_partitions=%d feat_tile=%s kernel=%s row_order=heaviest_first device=%s"
                % (layout, self._num_rows, self._num_cols, self._nnz, d, nfp,
                   tile if tile else "auto",
                   "fg_spmm_dds_f32" if self._num_col_partitions > 1 else "fg_spmm_csr_f32",
                   self._device))

    # -- run ----------------------------------------------------------------------------
    def _launch(self, x, out):
        L = dev.lib()
        d = self._feat_shape[1]
        s = dev.stream_ptr(self._device)
        if self._num_col_partitions > 1:
            rc = L.fg_spmm_dds_f32(self._schedule, dev.ptr(self._adj_pos), dev.ptr(self._adj_idx),
                                   dev.ptr(self._adj_vals), dev.ptr(x), 0, dev.ptr(out), 0,
                                   self._num_rows, self._num_cols, self._nnz, d,
                                   self._num_col_partitions, self._feat_tile, s)
        else:
            rc = L.fg_spmm_csr_f32(self._schedule, dev.ptr(self._adj_pos), dev.ptr(self._adj_idx),
                                   dev.ptr(self._adj_vals), dev.ptr(x), 0, dev.ptr(out), 0,
                                   self._num_rows, self._num_cols, self._nnz, d,
                                   self._feat_tile, s)
        dev.check(rc)

    def run(self, inputs):
        """Enqueue the kernel on the current stream and return the module's output tensor
        (the same object every call, as the reference returns ``out_tvm``, :142-161)."""
        if self.out is None:
            raise RuntimeError("call build() before run()")
        dev.refuse_if_deferred_pending(self)
        (x,) = inputs
        dev.check_input(x, self._feat_shape, self._device, "source features")
        with torch.cuda.device(self._device):
            self._launch(x, self.out)
        return self.out

    def run_host(self, inputs, out=None, chunk=0, wait=True):
        """Host-buffer call: features in host memory (numpy array or CPU tensor, float32,
        contiguous; pinned memory gives full copy speed), result back in host memory.  Copies and
        kernels are pipelined over column windows by ``fg_spmm_csr_f32_host``.  ``out``: a CPU
        float32 tensor ``[num_rows, feat_len]`` to fill (allocated pinned if omitted).  Returns it.
        ``wait=False``: return at once; the tensor is complete after ``featgraph_b200.host_sync()``
        (lets this call's copy-out overlap the next call; using this module again before that raises)."""
        if self.out is None:
            raise RuntimeError("call build() before run_host()")
        dev.refuse_if_deferred_pending(self)
        (x,) = inputs
        xt = torch.from_numpy(x) if isinstance(x, np.ndarray) else x
        if xt.device.type != "cpu" or xt.dtype != torch.float32 or not xt.is_contiguous() \
                or tuple(xt.shape) != tuple(self._feat_shape):
            raise ValueError("run_host wants a contiguous float32 host array of shape %s" % (self._feat_shape,))
        d = self._feat_shape[1]
        if out is None:
            out = torch.empty((self._num_rows, d), dtype=torch.float32).pin_memory()
        if out.device.type != "cpu" or out.dtype != torch.float32 or not out.is_contiguous() \
                or tuple(out.shape) != (self._num_rows, d):
            raise ValueError("out must be a contiguous float32 host tensor of shape %s" % ((self._num_rows, d),))
        with torch.cuda.device(self._device):
            if self._num_col_partitions > 1:
                # DDS layout: plain copy in, run, copy out
                out.copy_(self.run([xt.to(self._device, non_blocking=True)]))
                return out
            if self._x_staging is None or tuple(self._x_staging.shape) != tuple(self._feat_shape):
                self._x_staging = torch.empty(self._feat_shape, dtype=torch.float32, device=self._device)
            dev.check(dev.lib().fg_spmm_csr_f32_host(
                self._schedule, dev.ptr(self._adj_pos), dev.ptr(self._adj_idx), dev.ptr(self._adj_vals),
                ctypes.c_void_p(xt.data_ptr()), ctypes.c_void_p(out.data_ptr()), dev.ptr(self._x_staging),
                dev.ptr(self.out), self._num_rows, self._num_cols, self._nnz, d, int(chunk),
                0 if wait else 1, dev.stream_ptr(self._device)))
            if not wait:
                self._deferred_epoch = dev.sync_epoch(self._device)
        return out

    def measure_average_time(self, inputs, num_runs):
        """Mean seconds per call over ``num_runs`` back-to-back calls (reference :163-186)."""
        self.run(inputs)
        return dev.time_calls(lambda: self._launch(inputs[0], self.out), self._device, num_runs)

    @property
    def device_input(self):
        """The device copy of the features of the last ``run_host`` call (complete once the work enqueued by that
        call has run on the current stream): hand it to ``VanillaSDDMM*.run_host`` as the column-side matrix to
        score the same features without uploading them again."""
        return self._x_staging

    @property
    def ctx(self):
        """The device the module runs on (a ``torch.device``)."""
        return self._device

    @property
    def target(self):
        return self._target

    @property
    def row_order(self):
        """int32 device tensor: rows in the order the kernel visits them."""
        L = dev.lib()
        p = L.fg_row_schedule_order(self._schedule)
        n = self._num_rows
        if n == 0 or not p:
            return torch.empty(0, dtype=torch.int32, device=self._device)
        torch.cuda.current_stream(self._device).synchronize()
        return dev.view_device_int32(p, n, self._device).clone()


class VanillaSpMMx86(SpMMbase):
    """The x86 class of the reference (python/featgraph/module/spmm.py:197-209): column
    partitioning (DDS) and feature partitioning knobs, with its summation order."""

    _compute_keys = ("num_feat_partitions",)
    _schedule_keys = ("feat_tile",)

    def __init__(self, adj_scipy, num_col_partitions=1, device=None):
        super().__init__(adj_scipy, num_col_partitions, device)

    def _register(self):
        self._target = "llvm"


class VanillaSpMMcuda(SpMMbase):
    """The CUDA class of the reference (python/featgraph/module/spmm.py:212-220): plain CSR.
    ``num_cuda_blocks`` / ``num_threads_per_cuda_block`` are accepted and have no effect:
    rows map to thread blocks through the row schedule."""

    _compute_keys = ()
    _schedule_keys = ("num_cuda_blocks", "num_threads_per_cuda_block", "feat_tile")

    def __init__(self, adj_scipy, device=None, long_row_threshold=0):
        super().__init__(adj_scipy, 1, device, long_row_threshold)

    def _register(self):
        self._target = "cuda"
