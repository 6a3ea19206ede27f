"""Seeded synthetic graphs and features with the shapes the benchmarks are quoted on.

The reference benchmarks load the Reddit adjacency from a .npz produced by
benchmark/download_reddit_dataset.py:9-17 (needs a download); these generators make
stand-ins of the same size and sparsity pattern class.  Output: scipy CSR with int32
index arrays and all-ones float32 values (as that script stores them, :11,16), and
float32 feature matrices uniform in [-1, 1).  Everything is a pure function of the
seed (see csrc/graphgen.cpp), independent of thread count.
"""
import ctypes

import numpy as np
import scipy.sparse

from . import build as _build

_lib = None
_u64, _i64, _i32 = ctypes.c_uint64, ctypes.c_int64, ctypes.c_int32


def _L():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(_build.build_graphgen())
        L.fg_gen_num_threads.restype = ctypes.c_int
        L.fg_gen_uniform_f32.argtypes = [_u64, _i64, ctypes.c_void_p]
        L.fg_gen_uniform_f32.restype = None
        L.fg_gen_uniform_f64.argtypes = [_u64, _i64, ctypes.c_void_p]
        L.fg_gen_uniform_f64.restype = None
        L.fg_gen_neighbors.argtypes = [_u64, _i64, _i64, _i64, ctypes.c_void_p, ctypes.c_void_p]
        L.fg_gen_neighbors.restype = ctypes.c_int
        L.fg_gen_rmat_csr.argtypes = [_u64, _i32, _i64, ctypes.c_double, ctypes.c_double,
                                      ctypes.c_double, ctypes.c_void_p, ctypes.c_void_p]
        L.fg_gen_rmat_csr.restype = _i64
        _lib = L
    return _lib


def uniform_features(shape, seed, out=None):
    """float32 array of ``shape`` with values 2*u - 1, u a 24-bit uniform in [0, 1)."""
    if out is None:
        out = np.empty(shape, dtype=np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous
    _L().fg_gen_uniform_f32(int(seed), int(out.size), out.ctypes.data)
    return out


def _uniform_f64(count, seed):
    out = np.empty(count, dtype=np.float64)
    _L().fg_gen_uniform_f64(int(seed), int(count), out.ctypes.data)
    return out


def _csr_from_degrees(deg, n_cols, seed, row_offset=0):
    """CSR whose row r has ``deg[r]`` sorted distinct neighbours; ``row_offset`` is the global id of
    row 0, so a slice of a larger graph's rows can be generated alone."""
    n = deg.shape[0]
    indptr = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(deg, out=indptr[1:])
    nnz = int(indptr[-1])
    assert nnz < 2 ** 31, "int32 CSR only"
    indices = np.empty(nnz, dtype=np.int32)
    rc = _L().fg_gen_neighbors(int(seed), int(row_offset), n, int(n_cols), indptr.ctypes.data,
                                indices.ctypes.data)
    if rc != 0:
        raise ValueError("a row asks for more neighbours than there are columns")
    data = np.ones(nnz, dtype=np.float32)
    adj = scipy.sparse.csr_matrix((data, indices, indptr.astype(np.int32)), shape=(n, int(n_cols)))
    adj.has_sorted_indices = True
    return adj


def fixed_degree_graph(n, degree, seed, n_cols=None):
    """``n`` rows with exactly ``degree`` distinct uniform neighbours each, sorted CSR."""
    deg = np.full(n, int(degree), dtype=np.int64)
    return _csr_from_degrees(deg, n if n_cols is None else n_cols, seed)


def power_law_degrees(n, total_edges, seed, exponent=2.0, kmin=1, kmax=20000):
    """Per-row degrees: iid draws from p(k) ~ k^-exponent on [kmin, kmax], multiplied by
    the largest scale s such that sum(clip(floor(s*raw), kmin, kmax)) <= total_edges, then
    +1 on rows (in a seeded random order, only rows still below kmax) until the sum is exact."""
    kmax = min(int(kmax), int(n))
    ks = np.arange(kmin, kmax + 1, dtype=np.float64)
    cdf = np.cumsum(ks ** (-float(exponent)))
    cdf /= cdf[-1]
    raw = (np.searchsorted(cdf, _uniform_f64(n, seed), side="right") + kmin).astype(np.float64)
    raw = np.minimum(raw, kmax)

    def total(s):
        return int(np.clip(np.floor(s * raw), kmin, kmax).sum())

    assert n * kmin <= total_edges <= n * kmax, "edge total unreachable with these bounds"
    lo, hi = 0.0, float(kmax)
    for _ in range(200):
        mid = 0.5 * (lo + hi)
        if total(mid) <= total_edges:
            lo = mid
        else:
            hi = mid
    deg = np.clip(np.floor(lo * raw), kmin, kmax).astype(np.int64)
    order = np.argsort(_uniform_f64(n, seed + 7919), kind="stable")
    short = int(total_edges - deg.sum())
    while short > 0:
        cand = order[deg[order] < kmax][:short]
        assert cand.size > 0
        deg[cand] += 1
        short -= cand.size
    return deg


def power_law_graph(n, total_edges, seed, exponent=2.0, kmin=1, kmax=20000, rows=None):
    """``n`` x ``n`` sorted CSR with exactly ``total_edges`` nonzeros and power-law row degrees.
    ``rows=(lo, hi)`` returns only that row slice (shape ``(hi-lo, n)``), identical to slicing the
    whole graph."""
    deg = power_law_degrees(n, total_edges, seed, exponent, kmin, kmax)
    if rows is None:
        return _csr_from_degrees(deg, n, seed + 1)
    lo, hi = rows
    return _csr_from_degrees(deg[lo:hi], n, seed + 1, row_offset=lo)


def rmat_graph(scale, edge_factor, seed, a=0.57, b=0.19, c=0.19):
    """R-MAT graph on 2^scale vertices from ``edge_factor * 2^scale`` generated edges;
    self-loops and duplicates removed, sorted CSR.  ``adj.nnz`` is what survived."""
    n = 1 << int(scale)
    n_edges = int(edge_factor) * n
    assert n_edges < 2 ** 31, "int32 CSR only"
    indptr = np.empty(n + 1, dtype=np.int32)
    indices = np.empty(n_edges, dtype=np.int32)
    kept = _L().fg_gen_rmat_csr(int(seed), int(scale), n_edges, a, b, c, indptr.ctypes.data,
                                indices.ctypes.data)
    indices = indices[:kept].copy()
    adj = scipy.sparse.csr_matrix((np.ones(kept, dtype=np.float32), indices, indptr), shape=(n, n))
    adj.has_sorted_indices = True
    return adj


# The named workloads.  Graph seeds 20200 + graph id; feature seeds = graph seed + 1000 (+1
# for a second matrix).
WORKLOADS = {
    "C0": dict(kind="fixed", n=10_000, degree=20, seed=20200, d=(64,)),
    "C1": dict(kind="fixed", n=100_000, degree=32, seed=20201, d=(128,)),
    "C2": dict(kind="powerlaw", n=232_965, nnz=114_615_892, seed=20202, d=(32, 64, 128, 256, 512)),
    "C4": dict(kind="rmat", scale=22, edge_factor=32, seed=20204, d=(128,)),
}


def workload_graph(name, shrink=1):
    """Adjacency of a named workload.  ``shrink`` > 1 divides node and edge counts (tests)."""
    w = WORKLOADS[name]
    if w["kind"] == "fixed":
        return fixed_degree_graph(w["n"] // shrink, w["degree"], w["seed"])
    if w["kind"] == "powerlaw":
        n = w["n"] // shrink
        return power_law_graph(n, w["nnz"] // (shrink * shrink) if shrink > 1 else w["nnz"], w["seed"],
                               kmax=20000 // shrink if shrink > 1 else 20000)
    if w["kind"] == "rmat":
        s = w["scale"] - int(np.log2(shrink)) if shrink > 1 else w["scale"]
        return rmat_graph(s, w["edge_factor"], w["seed"])
    raise KeyError(name)


def workload_features(name, n, d, which=0):
    return uniform_features((n, d), WORKLOADS[name]["seed"] + 1000 + which)
