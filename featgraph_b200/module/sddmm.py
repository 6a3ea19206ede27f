"""SDDMM modules: same lifecycle and names as python/featgraph/module/sddmm.py of the
reference, executed by hand-written sm_100a kernels through the C ABI.

Both classes run on the GPU.  ``VanillaSDDMMx86`` keeps the x86 class's 2-D partitioning
knobs (the edge list is regrouped tile by tile and ``edge_mapping`` undoes it) and its summation
order (bit-identical results); ``VanillaSDDMMcuda`` takes the edge list as given and sums each
dot product as a tree, as the reference's CUDA schedule does.
"""
import numpy as np
import torch

from ..placeholder import check_float32, static_shape
from ..util import util_partition_adj_coo_2d
from . import _device as dev


class SDDMMbase:
    """Counterpart of ``SDDMMbase`` (python/featgraph/module/sddmm.py:11-165)."""

    _compute_keys = ()
    _schedule_keys = ()
    _exact_by_default = False

    def __init__(self, adj_scipy, num_row_partitions=1, num_col_partitions=1, device=None):
        # COO in SDDMM-like kernels (reference :28-31)
        adj_coo = adj_scipy.tocoo() if adj_scipy.format != "coo" else adj_scipy
        self._num_rows, self._num_cols = adj_coo.shape
        assert num_row_partitions >= 1, "num_row_partitions should be larger than or equal to 1"
        assert num_col_partitions >= 1, "num_col_partitions should be larger than or equal to 1"
        self._num_row_partitions = int(num_row_partitions)
        # Kept from the reference (:37): the column-partition count is taken from the ROW
        # argument, so the tiling is always square in partition counts.
        self._num_col_partitions = int(num_row_partitions)
        self._target = None
        self._register()
        self._device = dev.resolve_device(device)
        if self._num_row_partitions > 1 or self._num_col_partitions > 1:
            edge_ids, rows, cols = util_partition_adj_coo_2d(
                adj_coo, self._num_row_partitions, self._num_col_partitions)
            self._edge_mapping = np.argsort(edge_ids)
        else:
            rows, cols = adj_coo.row, adj_coo.col
        if rows.dtype != np.int32 or cols.dtype != np.int32:
            raise TypeError("int32 COO index arrays are required (got %s / %s)" % (rows.dtype, cols.dtype))
        self._nnz = int(rows.shape[0])
        import ctypes
        with torch.cuda.device(self._device):
            self._adj_row = dev.upload(rows, self._device)
            self._adj_col = dev.upload(cols, self._device)
            sorted_flag = ctypes.c_int32(0)
            dev.check(dev.lib().fg_coo_validate(dev.ptr(self._adj_row), dev.ptr(self._adj_col),
                                                self._num_rows, self._num_cols, self._nnz,
                                                ctypes.byref(sorted_flag),
                                                dev.stream_ptr(self._device)))
        self._rows_sorted = int(sorted_flag.value)
        self._plans = {}   # column-block plans by block count (built on first use, freed with the module)
        self._plan = None  # the plan the current build() uses, or None: plain fg_sddmm_coo_f32
        self._shapes = None
        self._feat_tile = 0
        self._exact = False
        self._staging = None
        self.out = None

    def __del__(self):
        plans = getattr(self, "_plans", None) or {}
        for h in plans.values():
            if h is not None and h.value:
                try:
                    dev.lib().fg_sddmm_plan_destroy(h)
                except Exception:
                    pass
        self._plans = {}

    def _register(self):
        raise NotImplementedError("Please register target.")

    def _column_block_plan(self, parts):
        """The plan for ``parts`` column blocks (built once, kept), or None where the edge list is not in
        CSR order (rows non-decreasing, column ids ascending within a row) and no plan can be built."""
        import ctypes
        if parts not in self._plans:
            handle = ctypes.c_void_p()
            with torch.cuda.device(self._device):
                rc = dev.lib().fg_sddmm_plan_create(dev.ptr(self._adj_row), dev.ptr(self._adj_col), self._num_rows,
                                                    self._num_cols, self._nnz, int(parts),
                                                    dev.stream_ptr(self._device), ctypes.byref(handle))
            if rc == 1 and b"CSR order" in dev.lib().fg_last_error():
                self._plans[parts] = None  # e.g. unsorted column ids inside rows: the plain call serves
            else:
                dev.check(rc)
                self._plans[parts] = handle
        return self._plans[parts]

    def _plan_args(self, input_placeholders, compute_args, schedule_args):
        compute_args = dict(compute_args or {})
        schedule_args = dict(schedule_args or {})
        for k in compute_args:
            if k not in self._compute_keys:
                raise TypeError("unexpected compute argument %r" % (k,))
        for k in schedule_args:
            if k not in self._schedule_keys:
                raise TypeError("unexpected schedule argument %r" % (k,))
        if len(input_placeholders) != 2:
            raise TypeError("SDDMM takes two inputs (column-side and row-side features)")
        src_shape = static_shape(input_placeholders[0])
        dst_shape = static_shape(input_placeholders[1])
        check_float32(input_placeholders[0])
        check_float32(input_placeholders[1])
        if len(src_shape) != 2 or len(dst_shape) != 2:
            raise ValueError("feature matrices must be 2-D")
        assert dst_shape[1] == src_shape[1], "dimension mismatch"
        # The first matrix is gathered by COLUMN id, the second by ROW id
        # (python/featgraph/op/vanilla_sddmm.py:47; tests/test_module_sddmm.py:18-19).
        if src_shape[0] != self._num_cols or dst_shape[0] != self._num_rows:
            raise ValueError("expected shapes [%d, d] and [%d, d], got %s and %s"
                             % (self._num_cols, self._num_rows, src_shape, dst_shape))
        d = src_shape[1]
        nfp = int(compute_args.get("num_feat_partitions", schedule_args.get("num_feat_partitions", 1)))
        if nfp < 1 or d % nfp != 0:
            raise ValueError("feat_len %d is not divisible by num_feat_partitions %d" % (d, nfp))
        self._check_schedule(schedule_args, nfp)
        tile = int(schedule_args.get("feat_tile", 0))
        if tile == 0 and nfp > 1:
            # the reference's feature tiling knob doubles as the L2 tile width when it is usable
            f = d // nfp
            if 4 <= f <= 512 and (f & (f - 1)) == 0:
                tile = f
        self._planned_tile = tile
        self._planned_exact = bool(schedule_args.get("exact", self._exact_by_default))
        # column blocks: 0 = let the library decide, 1 = never, P = that many
        self._planned_parts = int(schedule_args.get("col_blocks", 0))
        if self._planned_parts < 0:
            raise ValueError("col_blocks must be >= 0")
        return src_shape, dst_shape, d, nfp

    def _check_schedule(self, schedule_args, nfp):
        pass

    def build(self, input_placeholders, compute_args, schedule_args):
        """Fix the feature shapes and allocate the (reused) per-edge output (reference :72-92).
        ``schedule_args['exact'] = True`` selects the kernel that sums every dot product in the x86
        loop's order (bit-identical to it, three to four times slower); ``feat_tile`` sets the L2 tile width;
        ``col_blocks`` the number of column blocks of the one-pass traversal (0 = the library decides, 1 = off)."""
        src_shape, dst_shape, d, _ = self._plan_args(input_placeholders, compute_args, schedule_args)
        self._shapes = (src_shape, dst_shape)
        self._feat_tile = self._planned_tile
        self._exact = self._planned_exact
        # One pass over column blocks where the column-side matrix is too large for L2 (and no tile width
        # or exact order was asked for): needs a CSR-ordered edge list, else the tiled call serves.
        self._plan = None
        parts = self._planned_parts
        if parts == 0 and not self._exact and self._feat_tile == 0 and self._rows_sorted:
            parts = int(dev.lib().fg_sddmm_auto_partitions(self._num_rows, self._num_cols, self._nnz, d))
        if parts > 1 and not self._exact and self._rows_sorted and d % 4 == 0 and d <= 512:
            self._plan = self._column_block_plan(parts)
        self.out = torch.zeros((self._nnz,), dtype=torch.float32, device=self._device)

    def lower_to_ir(self, input_placeholders, compute_args, schedule_args):
        """Text description of what ``build`` + ``run`` would launch (reference :94-113)."""
        _, _, d, nfp = self._plan_args(input_placeholders, compute_args, schedule_args)
        return ("featgraph_b200 sddmm: rows=%d cols=%d nnz=%d feat_len=%d num_feat_partitions=%d "
                "edge_order=%s rows_sorted=%d kernel=%s device=%s"
                % (self._num_rows, self._num_cols, self._nnz, d, nfp,
                   "2d(%dx%d)" % (self._num_row_partitions, self._num_col_partitions)
                   if self._num_row_partitions > 1 else "as_given", self._rows_sorted,
                   "fg_sddmm_coo_f32_exact" if self._planned_exact else
                   "fg_sddmm_coo_f32 (or _planned over column blocks where the matrix exceeds L2)", self._device))

    def _launch(self, src, dst, out):
        d = self._shapes[0][1]
        if self._exact:
            dev.check(dev.lib().fg_sddmm_coo_f32_exact(dev.ptr(self._adj_row), dev.ptr(self._adj_col),
                                                       dev.ptr(src), 0, dev.ptr(dst), 0, dev.ptr(out),
                                                       self._num_rows, self._num_cols, self._nnz, d, 0,
                                                       dev.stream_ptr(self._device)))
            return
        if self._plan is not None:
            dev.check(dev.lib().fg_sddmm_coo_f32_planned(self._plan, dev.ptr(self._adj_col), dev.ptr(src), 0,
                                                         dev.ptr(dst), 0, dev.ptr(out), self._num_rows,
                                                         self._num_cols, self._nnz, d, 0,
                                                         dev.stream_ptr(self._device)))
            return
        dev.check(dev.lib().fg_sddmm_coo_f32(dev.ptr(self._adj_row), dev.ptr(self._adj_col),
                                             dev.ptr(src), 0, dev.ptr(dst), 0, dev.ptr(out),
                                             self._num_rows, self._num_cols, self._nnz, d,
                                             self._rows_sorted, 0, self._feat_tile,
                                             dev.stream_ptr(self._device)))

    def run(self, inputs):
        """Enqueue the kernel on the current stream; returns the module's output tensor (the
        same object every call, reference :115-129).  Argument order: [column-side, row-side]."""
        if self.out is None:
            raise RuntimeError("call build() before run()")
        dev.refuse_if_deferred_pending(self)
        src, dst = inputs
        dev.check_input(src, self._shapes[0], self._device, "column-side features")
        dev.check_input(dst, self._shapes[1], self._device, "row-side features")
        with torch.cuda.device(self._device):
            self._launch(src, dst, self.out)
        return self.out

    def run_host(self, inputs, out=None, chunk=0, wait=True):
        """Host-buffer call: both feature matrices in host memory (numpy or CPU tensors, float32,
        contiguous; pinned for full copy speed), per-edge result back in host memory, copies
        pipelined against the kernels by ``fg_sddmm_coo_f32_host``.  Returns the host tensor.
        ``wait=False``: return at once; the tensor is complete after ``featgraph_b200.host_sync()``
        (lets this call's copy-out overlap the next call; using this module again before that raises)."""
        if self.out is None:
            raise RuntimeError("call build() before run_host()")
        dev.refuse_if_deferred_pending(self)
        ts = [torch.from_numpy(x) if isinstance(x, np.ndarray) else x for x in inputs]
        # The column-side matrix may already be on the device (a CUDA tensor of the right shape, e.g.
        # ``VanillaSpMM*.device_input`` after that module's run_host on the same features): it is then used where it
        # is, not copied - a layer that runs both ops uploads its features once.
        src_resident = ts[0].device == self._device
        for k, (t, shape) in enumerate(zip(ts, self._shapes)):
            on_host = t.device.type == "cpu"
            if not (on_host or (k == 0 and src_resident)) or t.dtype != torch.float32 or not t.is_contiguous() \
                    or tuple(t.shape) != tuple(shape):
                raise ValueError("run_host wants contiguous float32 host arrays of shapes %s (the first may be a "
                                 "tensor on the module's device)" % (self._shapes,))
        if out is None:
            out = torch.empty((self._nnz,), dtype=torch.float32).pin_memory()
        if out.device.type != "cpu" or out.dtype != torch.float32 or tuple(out.shape) != (self._nnz,):
            raise ValueError("out must be a float32 host tensor of shape (%d,)" % self._nnz)
        import ctypes
        d = self._shapes[0][1]
        with torch.cuda.device(self._device):
            if self._staging is None or tuple(self._staging[1].shape) != tuple(self._shapes[1]) \
                    or (not src_resident and tuple(self._staging[0].shape) != tuple(self._shapes[0])):
                self._staging = (torch.empty(self._shapes[0] if not src_resident else (0, d), dtype=torch.float32,
                                             device=self._device),
                                 torch.empty(self._shapes[1], dtype=torch.float32, device=self._device))
            src_dev = ts[0] if src_resident else self._staging[0]
            if src_resident and self._plan is not None and chunk == 0:
                # column side on the device, matrix larger than L2: the one-pass kernel over column blocks
                dev.check(dev.lib().fg_sddmm_coo_f32_planned_host(
                    self._plan, dev.ptr(self._adj_col), dev.ptr(src_dev), ctypes.c_void_p(ts[1].data_ptr()),
                    ctypes.c_void_p(out.data_ptr()), dev.ptr(self._staging[1]), dev.ptr(self.out), self._num_rows,
                    self._num_cols, self._nnz, d, 0 if wait else 1, dev.stream_ptr(self._device)))
                if not wait:
                    self._deferred_epoch = dev.sync_epoch(self._device)
                return out
            dev.check(dev.lib().fg_sddmm_coo_f32_host(
                dev.ptr(self._adj_row), dev.ptr(self._adj_col),
                ctypes.c_void_p(0) if src_resident else ctypes.c_void_p(ts[0].data_ptr()),
                ctypes.c_void_p(ts[1].data_ptr()), ctypes.c_void_p(out.data_ptr()), dev.ptr(src_dev),
                dev.ptr(self._staging[1]), dev.ptr(self.out), self._num_rows, self._num_cols, self._nnz, d,
                self._rows_sorted, int(chunk), 0 if wait else 1, dev.stream_ptr(self._device)))
            if not wait:
                self._deferred_epoch = dev.sync_epoch(self._device)
        return out

    def measure_average_time(self, inputs, num_runs):
        """Mean seconds per call over ``num_runs`` back-to-back calls (reference :131-150)."""
        self.run(inputs)
        return dev.time_calls(lambda: self._launch(inputs[0], inputs[1], self.out), self._device,
                              num_runs)

    @property
    def edge_mapping(self):
        """Permutation that puts the output back into the caller's edge order:
        ``out[edge_mapping]`` (reference :152-157)."""
        assert self._target != 'cuda', "no graph partitioning on cuda, no edge_mapping"
        assert self._num_row_partitions > 1 or self._num_col_partitions > 1, \
            "no graph partitioning, no edge_mapping"
        return self._edge_mapping

    @property
    def ctx(self):
        return self._device

    @property
    def target(self):
        return self._target


class VanillaSDDMMx86(SDDMMbase):
    """The x86 class of the reference (python/featgraph/module/sddmm.py:168-176).  It keeps the x86
    path's arithmetic: by default the exact-order kernel runs, so results are bit-identical to the
    x86 loop (``schedule_args={'exact': False}`` selects the faster tree-summed kernel)."""

    _compute_keys = ("num_feat_partitions",)
    _exact_by_default = True
    _schedule_keys = ("num_feat_partitions", "feat_tile", "exact", "col_blocks")

    def __init__(self, adj_scipy, num_row_partitions=1, num_col_partitions=1, device=None):
        super().__init__(adj_scipy, num_row_partitions, num_col_partitions, device)

    def _register(self):
        self._target = "llvm"


class VanillaSDDMMcuda(SDDMMbase):
    """The CUDA class of the reference (python/featgraph/module/sddmm.py:179-187).
    ``num_cuda_blocks`` is checked as the reference's schedule checks it
    (python/featgraph/op/vanilla_sddmm.py:79-82) and otherwise has no effect."""

    _compute_keys = ()
    _schedule_keys = ("num_feat_partitions", "num_cuda_blocks", "feat_tile", "exact", "col_blocks")

    def __init__(self, adj_scipy, device=None):
        super().__init__(adj_scipy, 1, 1, device)

    def _register(self):
        self._target = "cuda"

    def _check_schedule(self, schedule_args, nfp):
        assert nfp == 1, "cuda schedule for sddmm does not support feat dimension tiling, " \
                         "which requires cross-cuda-block reduction and atomic operations."
        blocks = schedule_args.get("num_cuda_blocks", 8192)
        if "num_cuda_blocks" in schedule_args:
            assert blocks <= self._nnz, "num_cuda_blocks must be smaller than num_edges, " \
                                        "which is {}.".format(self._nnz)
