"""Aggregate-then-score: one GCN-style layer step, H = A.X followed by out[e] = dot(H[row e], Y[col e]).

A caller of the reference runs this as two built functions back to back - ``VanillaSpMM*.run([X])``
(python/featgraph/module/spmm.py:142-161), then ``VanillaSDDMM*.run([Y, H])``
(python/featgraph/module/sddmm.py:115-129).  ``AggregateThenScore`` has the same lifecycle (construct from a
scipy adjacency, ``build``, ``run``) and does both in one pass over the rows: the group of lanes that has
just finished a row of H still holds it in registers and scores the row's edges at once
(``fg_spmm_sddmm_fused_f32``).  H is bit-identical to ``VanillaSpMMcuda``; the scores agree with
``VanillaSDDMMcuda`` on the CSR-ordered edge list to fp32 rounding of d terms.
"""
import ctypes

import numpy as np
import torch

from ..placeholder import check_float32, static_shape
from . import _device as dev

MAX_FEAT_LEN = 128  # a whole row of H lives in one lane group's registers


class AggregateThenScore:
    """``run([X, Y]) -> (H, scores)`` for a square or rectangular adjacency [num_rows, num_cols]:
    X and Y are [num_cols, d] (both gathered by column id), H is [num_rows, d], scores has one entry per
    nonzero in CSR order.  d <= 128, a multiple of 4."""

    def __init__(self, adj_scipy, device=None, long_row_threshold=0):
        adj_csr = adj_scipy.tocsr() if adj_scipy.format != "csr" else adj_scipy
        self._num_rows, self._num_cols = adj_csr.shape
        self._device = dev.resolve_device(device)
        self._nnz = int(adj_csr.indices.shape[0])
        if adj_csr.indptr.dtype != np.int32 or adj_csr.indices.dtype != np.int32:
            raise TypeError("int32 CSR index arrays are required (got %s / %s)"
                            % (adj_csr.indptr.dtype, adj_csr.indices.dtype))
        if adj_csr.data.dtype != np.float32:
            raise TypeError("float32 adjacency values are required, got %s" % adj_csr.data.dtype)
        unit_values = bool(self._nnz == 0 or np.all(adj_csr.data == np.float32(1.0)))
        L = dev.lib()
        with torch.cuda.device(self._device):
            self._indptr = dev.upload(adj_csr.indptr, self._device)
            self._indices = dev.upload(adj_csr.indices, self._device)
            self._vals = None if unit_values else dev.upload(adj_csr.data, self._device)
            dev.check(L.fg_csr_validate(dev.ptr(self._indptr), dev.ptr(self._indices), self._num_rows,
                                        self._num_cols, self._nnz, dev.stream_ptr(self._device)))
            self._schedule = ctypes.c_void_p()
            dev.check(L.fg_row_schedule_create(dev.ptr(self._indptr), self._num_rows, int(long_row_threshold),
                                               dev.stream_ptr(self._device), ctypes.byref(self._schedule)))
        self._feat_shape = None
        self.out = None     # H
        self.scores = None  # per-edge output

    def __del__(self):
        sched = getattr(self, "_schedule", None)
        if sched is not None and sched.value:
            try:
                dev.lib().fg_row_schedule_destroy(sched)
            except Exception:
                pass
            self._schedule = None

    def build(self, input_placeholders, compute_args=None, schedule_args=None):
        """Fix the feature shape ([num_cols, d] for both inputs) and allocate the reused outputs."""
        if compute_args or schedule_args:
            raise TypeError("AggregateThenScore takes no compute or schedule arguments")
        if len(input_placeholders) != 2:
            raise TypeError("two inputs: the features to aggregate and the features to score against")
        shapes = [static_shape(p) for p in input_placeholders]
        for p in input_placeholders:
            check_float32(p)
        if shapes[0] != shapes[1] or len(shapes[0]) != 2 or shapes[0][0] != self._num_cols:
            raise ValueError("both feature matrices must be [num_cols=%d, feat_len], got %s and %s"
                             % (self._num_cols, shapes[0], shapes[1]))
        d = shapes[0][1]
        if d > MAX_FEAT_LEN or d % 4 != 0:
            raise ValueError("feat_len %d: the fused step takes a multiple of 4 up to %d "
                             "(run VanillaSpMMcuda then VanillaSDDMMcuda otherwise)" % (d, MAX_FEAT_LEN))
        self._feat_shape = shapes[0]
        self.out = torch.zeros((self._num_rows, d), dtype=torch.float32, device=self._device)
        self.scores = torch.zeros((self._nnz,), dtype=torch.float32, device=self._device)

    def _launch(self, x, y):
        d = self._feat_shape[1]
        dev.check(dev.lib().fg_spmm_sddmm_fused_f32(
            self._schedule, dev.ptr(self._indptr), dev.ptr(self._indices), dev.ptr(self._vals), dev.ptr(x), 0,
            dev.ptr(y), 0, dev.ptr(self.out), 0, dev.ptr(self.scores), self._num_rows, self._num_cols, self._nnz, d,
            dev.stream_ptr(self._device)))

    def run(self, inputs):
        """Enqueue the step on the current stream; returns ``(H, scores)``, the same tensors every call."""
        if self.out is None:
            raise RuntimeError("call build() before run()")
        x, y = inputs
        dev.check_input(x, self._feat_shape, self._device, "features to aggregate")
        dev.check_input(y, self._feat_shape, self._device, "features to score against")
        with torch.cuda.device(self._device):
            self._launch(x, y)
        return self.out, self.scores

    def measure_average_time(self, inputs, num_runs):
        """Mean seconds per call over ``num_runs`` back-to-back calls after one warm-up."""
        self.run(inputs)
        return dev.time_calls(lambda: self._launch(inputs[0], inputs[1]), self._device, num_runs)

    @property
    def ctx(self):
        return self._device
