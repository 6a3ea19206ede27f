"""CPU oracle for the vanilla SpMM / SDDMM hot path (TEST INFRASTRUCTURE ONLY).

Python face of ``featgraph_oracle.c``: loads ``oracle/_ref/libfeatgraph_oracle.so``
(building it with ``make`` when it is missing and a C compiler is present) and wraps
each function for numpy arrays.  Only the tests, the smoke check and the benchmark's
CPU-baseline leg import this package; the shipped library never does.

Parity: bit-identical to the reference's own SpMM / SDDMM compute definitions compiled by a TVM
build (fixtures tests/golden/*_reference_tvm.npz; see the header of ``featgraph_oracle.c``);
index arithmetic and accumulation order follow python/featgraph/op/vanilla_spmm.py:41-62,195-224
and op/vanilla_sddmm.py:43-62.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "_ref", "libfeatgraph_oracle.so")
_lib = None

_i64, _i32, _int = ctypes.c_int64, ctypes.c_int32, ctypes.c_int
_pi32 = ctypes.POINTER(ctypes.c_int32)
_pf32 = ctypes.POINTER(ctypes.c_float)


def build(force=False):
    """Compile the C oracle into oracle/_ref/ (no-op when it is already there)."""
    src = os.path.join(_HERE, "featgraph_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B"], check=True, capture_output=True)
    return _SO


def lib():
    global _lib
    if _lib is None:
        build()
        L = ctypes.CDLL(_SO)
        L.fgo_num_threads.restype = _int
        L.fgo_spmm_csr_x86.argtypes = [_i64, _i64, _i32, _i32, _pi32, _pi32, _pf32, _pf32, _pf32, _int, _int]
        L.fgo_spmm_csr_dynamic.argtypes = [_i64, _i32, _pi32, _pi32, _pf32, _pf32, _pf32, _int]
        L.fgo_spmm_dds_x86.argtypes = [_i64, _i64, _i32, _i32, _i32, _pi32, _pi32, _pf32, _pf32, _pf32, _int]
        L.fgo_sddmm_x86.argtypes = [_i64, _i32, _i32, _pi32, _pi32, _pf32, _pf32, _pf32, _int, _int]
        for f in (L.fgo_spmm_csr_x86, L.fgo_spmm_csr_dynamic, L.fgo_spmm_dds_x86, L.fgo_sddmm_x86):
            f.restype = _int
        _lib = L
    return _lib


def num_threads():
    return int(lib().fgo_num_threads())


def _i(a):
    a = np.ascontiguousarray(a, dtype=np.int32)
    return a, a.ctypes.data_as(_pi32)


def _f(a):
    a = np.ascontiguousarray(a, dtype=np.float32)
    return a, a.ctypes.data_as(_pf32)


def spmm_csr(indptr, indices, vals, X, num_feat_partitions=1, use_fma=False, with_copies=False,
             dynamic=False, out=None):
    """Out = A . X the way the reference's x86 CSR schedule sums it
    (python/featgraph/op/vanilla_spmm.py:41-62, schedule :65-80)."""
    X, pX = _f(X)
    n_cols, d = X.shape
    indptr, pip = _i(indptr)
    indices, pix = _i(indices)
    vals, pv = _f(vals)
    n_rows = indptr.shape[0] - 1
    assert d % num_feat_partitions == 0
    if out is None:
        out = np.empty((n_rows, d), dtype=np.float32)
    po = out.ctypes.data_as(_pf32)
    if dynamic:
        rc = lib().fgo_spmm_csr_dynamic(n_rows, d, pip, pix, pv, pX, po, int(use_fma))
    else:
        rc = lib().fgo_spmm_csr_x86(n_rows, n_cols, d, num_feat_partitions, pip, pix, pv, pX, po,
                                    int(use_fma), int(with_copies))
    if rc != 0:
        raise MemoryError("oracle spmm: scratch allocation failed")
    return out


def spmm_dds(s1_pos, s1_idx, vals, X, n_rows, num_col_partitions, num_feat_partitions=1,
             use_fma=False):
    """DDS variant: per column partition partial sums, added in partition order
    (python/featgraph/op/vanilla_spmm.py:195-224, schedule :227-246)."""
    X, pX = _f(X)
    n_cols, d = X.shape
    s1_pos, pp = _i(s1_pos)
    s1_idx, pi = _i(s1_idx)
    vals, pv = _f(vals)
    assert s1_pos.shape[0] == num_col_partitions * (n_rows + 1)
    assert d % num_feat_partitions == 0
    out = np.empty((n_rows, d), dtype=np.float32)
    rc = lib().fgo_spmm_dds_x86(n_rows, n_cols, d, num_feat_partitions, num_col_partitions, pp, pi,
                                pv, pX, out.ctypes.data_as(_pf32), int(use_fma))
    assert rc == 0
    return out


def sddmm(row, col, src, dst, num_feat_partitions=1, use_fma=False, threads=1, out=None):
    """out[e] = sum_k src[col[e], k] * dst[row[e], k], k ascending, fp32
    (python/featgraph/op/vanilla_sddmm.py:43-62; single thread as at :66-74)."""
    src, ps = _f(src)
    dst, pd = _f(dst)
    row, pr = _i(row)
    col, pc = _i(col)
    d = src.shape[1]
    assert dst.shape[1] == d and d % num_feat_partitions == 0
    nnz = row.shape[0]
    if out is None:
        out = np.empty((nnz,), dtype=np.float32)
    rc = lib().fgo_sddmm_x86(nnz, d, num_feat_partitions, pr, pc, ps, pd,
                             out.ctypes.data_as(_pf32), int(use_fma), int(threads))
    assert rc == 0
    return out
