"""Helpers for the GPU parity tests: call the library through its C ABI on torch-owned memory."""
import ctypes

import numpy as np
import torch

from featgraph_b200 import _native


def dev(a, dtype=None):
    return torch.from_numpy(np.ascontiguousarray(a, dtype=dtype)).cuda()


def p(t):
    return ctypes.c_void_p(t.data_ptr()) if t is not None and t.numel() else ctypes.c_void_p(0)


def stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


class Schedule:
    def __init__(self, indptr_dev, n_rows, long_row_threshold=0):
        self.h = ctypes.c_void_p()
        _native.check(_native.lib().fg_row_schedule_create(p(indptr_dev), n_rows, long_row_threshold, stream(),
                                                           ctypes.byref(self.h)))

    def close(self):
        if self.h.value:
            _native.lib().fg_row_schedule_destroy(self.h)
            self.h = ctypes.c_void_p()

    def __del__(self):
        self.close()


GUARD = 64  # floats of NaN sentinel on either side of an output


def guarded(shape_numel):
    buf = torch.full((shape_numel + 2 * GUARD,), float("nan"), dtype=torch.float32, device="cuda")
    return buf, buf[GUARD:GUARD + shape_numel]


def guards_intact(buf):
    return bool(torch.isnan(buf[:GUARD]).all() and torch.isnan(buf[-GUARD:]).all())


def spmm_csr(indptr, indices, vals, x, feat_tile=0, use_schedule=True, check_guards=True, long_row_threshold=0):
    """fg_spmm_csr_f32 on numpy inputs; returns a numpy [n_rows, d]."""
    L = _native.lib()
    n_rows = len(indptr) - 1
    n_cols, d = x.shape
    ip, ix, xx = dev(indptr, np.int32), dev(indices, np.int32), dev(x, np.float32)
    vv = dev(vals, np.float32) if vals is not None else None  # None: unit values, no array
    buf, out = guarded(n_rows * d)
    sch = Schedule(ip, n_rows, long_row_threshold) if use_schedule else None
    _native.check(L.fg_spmm_csr_f32(sch.h if sch else None, p(ip), p(ix), p(vv), p(xx), 0, p(out), 0, n_rows, n_cols,
                                    len(indices), d, feat_tile, stream()))
    torch.cuda.synchronize()
    if check_guards:
        assert guards_intact(buf), "kernel wrote outside its output"
    res = out.cpu().numpy().reshape(n_rows, d)
    if sch:
        sch.close()
    return res


def spmm_dds(s1_pos, s1_idx, vals, x, n_rows, parts, indptr_for_schedule=None, feat_tile=0):
    L = _native.lib()
    n_cols, d = x.shape
    pp, ii, vv, xx = dev(s1_pos, np.int32), dev(s1_idx, np.int32), dev(vals, np.float32), dev(x, np.float32)
    buf, out = guarded(n_rows * d)
    sch = None
    if indptr_for_schedule is not None:
        sch = Schedule(dev(indptr_for_schedule, np.int32), n_rows)
    _native.check(L.fg_spmm_dds_f32(sch.h if sch else None, p(pp), p(ii), p(vv), p(xx), 0, p(out), 0, n_rows, n_cols,
                                    len(s1_idx), d, parts, feat_tile, stream()))
    torch.cuda.synchronize()
    assert guards_intact(buf), "kernel wrote outside its output"
    return out.cpu().numpy().reshape(n_rows, d)


def sddmm(row, col, src, dst, rows_sorted=0, feat_tile=0):
    L = _native.lib()
    n_cols, d = src.shape
    n_rows = dst.shape[0]
    rr, cc, ss, dd = dev(row, np.int32), dev(col, np.int32), dev(src, np.float32), dev(dst, np.float32)
    buf, out = guarded(len(row))
    _native.check(L.fg_sddmm_coo_f32(p(rr), p(cc), p(ss), 0, p(dd), 0, p(out), n_rows, n_cols, len(row), d,
                                     int(rows_sorted), 0, int(feat_tile), stream()))
    torch.cuda.synchronize()
    assert guards_intact(buf), "kernel wrote outside its output"
    return out.cpu().numpy()


def sddmm_exact(row, col, src, dst):
    L = _native.lib()
    n_cols, d = src.shape
    n_rows = dst.shape[0]
    rr, cc, ss, dd = dev(row, np.int32), dev(col, np.int32), dev(src, np.float32), dev(dst, np.float32)
    buf, out = guarded(len(row))
    _native.check(L.fg_sddmm_coo_f32_exact(p(rr), p(cc), p(ss), 0, p(dd), 0, p(out), n_rows, n_cols, len(row), d, 0,
                                           stream()))
    torch.cuda.synchronize()
    assert guards_intact(buf), "kernel wrote outside its output"
    return out.cpu().numpy()


class SddmmPlan:
    """fg_sddmm_plan over device row / col arrays (column blocks of ceil(n_cols / parts))."""

    def __init__(self, row_dev, col_dev, n_rows, n_cols, parts):
        self.h = ctypes.c_void_p()
        _native.check(_native.lib().fg_sddmm_plan_create(p(row_dev), p(col_dev), n_rows, n_cols, row_dev.numel(),
                                                         parts, stream(), ctypes.byref(self.h)))

    def close(self):
        if self.h.value:
            _native.lib().fg_sddmm_plan_destroy(self.h)
            self.h = ctypes.c_void_p()

    def __del__(self):
        self.close()


def sddmm_planned(row, col, src, dst, parts, accumulate_onto=None):
    """fg_sddmm_coo_f32_planned on numpy inputs (a CSR-ordered edge list); returns the numpy per-edge output."""
    L = _native.lib()
    n_cols, d = src.shape
    n_rows = dst.shape[0]
    rr, cc, ss, dd = dev(row, np.int32), dev(col, np.int32), dev(src, np.float32), dev(dst, np.float32)
    buf, out = guarded(len(row))
    if accumulate_onto is not None:
        out.copy_(torch.from_numpy(accumulate_onto).cuda())
    plan = SddmmPlan(rr, cc, n_rows, n_cols, parts)
    assert L.fg_sddmm_plan_partitions(plan.h) == parts
    _native.check(L.fg_sddmm_coo_f32_planned(plan.h, p(cc), p(ss), 0, p(dd), 0, p(out), n_rows, n_cols, len(row), d,
                                             1 if accumulate_onto is not None else 0, stream()))
    torch.cuda.synchronize()
    assert guards_intact(buf), "kernel wrote outside its output"
    plan.close()
    return out.cpu().numpy()
