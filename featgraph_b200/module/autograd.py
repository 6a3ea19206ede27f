"""Differentiable SpMM / SDDMM: the backward passes, composed from the same two kernels.

The reference checkout holds forward kernels only (its README, lines 9-11, points to a branch with
"generalized SpMM and generalized SDDMM" that is not part of it), yet a GNN layer trained on top of them
needs gradients.  Both backward passes are again an SpMM and an SDDMM on the same graph:

    out = A(w) . X          dX     = A(w)^T . dOut                      SpMM on the transposed adjacency
                            dw[e]  = dot(dOut[row e], X[col e])         SDDMM
    s[e] = dot(Src[col e], Dst[row e])
                            dDst   = A(g) . Src   with g = ds            SpMM, the incoming gradient as edge values
                            dSrc   = A(g)^T . Dst                       SpMM on the transposed adjacency

so ``GraphOps`` keeps the adjacency twice (CSR and the CSR of its transpose, with the permutation that carries
per-edge values from one order to the other) and calls the forward entry points for everything.  Sums run in
CSR order of whichever adjacency is walked: no atomics, the same gradient bits on every run.
"""
import ctypes

import numpy as np
import scipy.sparse
import torch

from . import _device as dev


class _Csr:
    """One orientation of the adjacency on the device: indptr, indices, a row schedule, COO rows."""

    def __init__(self, csr, device):
        self.n_rows, self.n_cols = csr.shape
        self.nnz = int(csr.nnz)
        L = dev.lib()
        with torch.cuda.device(device):
            self.indptr = dev.upload(csr.indptr.astype(np.int32), device)
            self.indices = dev.upload(csr.indices.astype(np.int32), device)
            self.rows = dev.upload(np.repeat(np.arange(self.n_rows, dtype=np.int32), np.diff(csr.indptr)), device)
            dev.check(L.fg_csr_validate(dev.ptr(self.indptr), dev.ptr(self.indices), self.n_rows, self.n_cols,
                                        self.nnz, dev.stream_ptr(device)))
            self.schedule = ctypes.c_void_p()
            dev.check(L.fg_row_schedule_create(dev.ptr(self.indptr), self.n_rows, 0, dev.stream_ptr(device),
                                               ctypes.byref(self.schedule)))

    def close(self):
        if self.schedule is not None and self.schedule.value:
            try:
                dev.lib().fg_row_schedule_destroy(self.schedule)
            except Exception:
                pass
            self.schedule = None


class GraphOps:
    """Differentiable ``spmm`` and ``sddmm`` on one adjacency [num_rows, num_cols] (structure only: edge
    values, if any, are an argument, so that they can carry gradients).

    ``spmm(x, edge_weight=None)``: x [num_cols, d] -> [num_rows, d]; ``edge_weight`` [nnz] in CSR order.
    ``sddmm(src, dst)``: src [num_cols, d] (gathered by column id), dst [num_rows, d] -> [nnz] in CSR order."""

    def __init__(self, adj_scipy, device=None):
        csr = adj_scipy.tocsr()
        csr.sort_indices()
        self._device = dev.resolve_device(device)
        self.num_rows, self.num_cols = csr.shape
        self.nnz = int(csr.nnz)
        # the transpose in CSR form, its nonzeros tagged with their position in the forward CSR order
        tagged = scipy.sparse.csr_matrix((np.arange(1, self.nnz + 1, dtype=np.int64), csr.indices, csr.indptr),
                                         shape=csr.shape).T.tocsr()
        tagged.sort_indices()
        self._fwd = _Csr(csr, self._device)
        self._bwd = _Csr(tagged, self._device)
        self._to_transposed = torch.from_numpy((tagged.data - 1).astype(np.int64)).to(self._device)

    def __del__(self):
        for side in ("_fwd", "_bwd"):
            obj = getattr(self, side, None)
            if obj is not None:
                obj.close()

    # ---- raw calls (no autograd) ----
    def _spmm(self, side, x, weight):
        x = x.contiguous()
        d = x.shape[1]
        out = torch.empty((side.n_rows, d), dtype=torch.float32, device=self._device)
        with torch.cuda.device(self._device):
            dev.check(dev.lib().fg_spmm_csr_f32(side.schedule, dev.ptr(side.indptr), dev.ptr(side.indices),
                                                dev.ptr(weight), dev.ptr(x), 0, dev.ptr(out), 0, side.n_rows,
                                                side.n_cols, side.nnz, d, 0, dev.stream_ptr(self._device)))
        return out

    def _sddmm(self, src, dst):
        src, dst = src.contiguous(), dst.contiguous()
        d = src.shape[1]
        out = torch.empty((self.nnz,), dtype=torch.float32, device=self._device)
        f = self._fwd
        with torch.cuda.device(self._device):
            dev.check(dev.lib().fg_sddmm_coo_f32(dev.ptr(f.rows), dev.ptr(f.indices), dev.ptr(src), 0, dev.ptr(dst), 0,
                                                 dev.ptr(out), f.n_rows, f.n_cols, f.nnz, d, 1, 0, 0,
                                                 dev.stream_ptr(self._device)))
        return out

    def _check(self, t, rows, what):
        if not isinstance(t, torch.Tensor) or t.device != self._device or t.dtype != torch.float32 or t.dim() != 2 \
                or t.shape[0] != rows:
            raise ValueError("%s must be a float32 tensor [%d, d] on %s" % (what, rows, self._device))

    # ---- generalized forms (forward only) ----
    REDUCE = {"max": 1, "min": 2, "mean": 3}
    EDGE_OP = {"add": 0, "sub": 1, "mul": 2}

    def spmm_reduce(self, x, reduce, edge_weight=None):
        """out[r] = reduce over row r's nonzeros of edge_weight[e] * x[col e], reduce in 'max' / 'min' / 'mean'
        (rows without nonzeros give 0).  Forward only."""
        self._check(x, self.num_cols, "x")
        x = x.contiguous()
        d = x.shape[1]
        f = self._fwd
        out = torch.empty((f.n_rows, d), dtype=torch.float32, device=self._device)
        with torch.cuda.device(self._device):
            dev.check(dev.lib().fg_spmm_csr_reduce_f32(dev.ptr(f.indptr), dev.ptr(f.indices), dev.ptr(edge_weight),
                                                       dev.ptr(x), 0, dev.ptr(out), 0, f.n_rows, f.n_cols, f.nnz, d,
                                                       self.REDUCE[reduce], dev.stream_ptr(self._device)))
        return out

    def edge_op(self, src, dst, op):
        """out[e, :] = src[col e, :] (op) dst[row e, :], op in 'add' / 'sub' / 'mul'; [nnz, d] in CSR order.
        Forward only."""
        self._check(src, self.num_cols, "src")
        self._check(dst, self.num_rows, "dst")
        src, dst = src.contiguous(), dst.contiguous()
        d = src.shape[1]
        f = self._fwd
        out = torch.empty((f.nnz, d), dtype=torch.float32, device=self._device)
        with torch.cuda.device(self._device):
            dev.check(dev.lib().fg_edge_binary_f32(dev.ptr(f.rows), dev.ptr(f.indices), dev.ptr(src), 0, dev.ptr(dst), 0,
                                                   dev.ptr(out), 0, f.n_rows, f.n_cols, f.nnz, d, self.EDGE_OP[op],
                                                   dev.stream_ptr(self._device)))
        return out

    # ---- differentiable calls ----
    def spmm(self, x, edge_weight=None):
        self._check(x, self.num_cols, "x")
        if edge_weight is not None and (edge_weight.shape != (self.nnz,) or edge_weight.dtype != torch.float32
                                        or edge_weight.device != self._device):
            raise ValueError("edge_weight must be a float32 tensor [%d] on %s" % (self.nnz, self._device))
        return _SpMM.apply(self, x, edge_weight)

    def sddmm(self, src, dst):
        self._check(src, self.num_cols, "src")
        self._check(dst, self.num_rows, "dst")
        if src.shape[1] != dst.shape[1]:
            raise ValueError("dimension mismatch")
        return _SDDMM.apply(self, src, dst)


class _SpMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ops, x, weight):
        ctx.ops = ops
        ctx.save_for_backward(x, weight)
        return ops._spmm(ops._fwd, x, None if weight is None else weight.contiguous())

    @staticmethod
    def backward(ctx, grad_out):
        ops = ctx.ops
        x, weight = ctx.saved_tensors
        grad_out = grad_out.contiguous()
        dx = dw = None
        if ctx.needs_input_grad[1]:
            wt = None if weight is None else weight.index_select(0, ops._to_transposed)
            dx = ops._spmm(ops._bwd, grad_out, wt)  # A(w)^T . dOut
        if weight is not None and ctx.needs_input_grad[2]:
            dw = ops._sddmm(x, grad_out)  # dot(x[col e], dOut[row e])
        return None, dx, dw


class _SDDMM(torch.autograd.Function):
    @staticmethod
    def forward(ctx, ops, src, dst):
        ctx.ops = ops
        ctx.save_for_backward(src, dst)
        return ops._sddmm(src, dst)

    @staticmethod
    def backward(ctx, grad_out):
        ops = ctx.ops
        src, dst = ctx.saved_tensors
        g = grad_out.contiguous()
        dsrc = ddst = None
        if ctx.needs_input_grad[1]:
            dsrc = ops._spmm(ops._bwd, dst, g.index_select(0, ops._to_transposed))  # A(g)^T . Dst
        if ctx.needs_input_grad[2]:
            ddst = ops._spmm(ops._fwd, src, g)  # A(g) . Src
        return None, dsrc, ddst
