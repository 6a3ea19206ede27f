"""Seeded random sweep over shapes, feature lengths, knobs and value kinds: SpMM bit-exact, SDDMM within
tolerance (default kernel) and bit-exact (exact-order kernel), all through the C ABI."""
import numpy as np
import pytest
import scipy.sparse as sp

from conftest import ATOL, RTOL

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("seed", range(12))
def test_random_cases(oracle, seed):
    import gpu_util as G
    from featgraph_b200 import graphgen
    from featgraph_b200.util import util_convert_csr_to_dds
    rng = np.random.default_rng(1000 + seed)
    for _ in range(4):
        n_rows = int(rng.integers(1, 700))
        n_cols = int(rng.integers(1, 900))
        d = int(rng.choice([1, 2, 4, 5, 8, 12, 16, 24, 32, 40, 64, 68, 96, 128, 160, 256, 260, 384, 512, 516]))
        kind = rng.choice(["uniform", "skewed", "empty-ish"])
        if kind == "uniform":
            adj = sp.random(n_rows, n_cols, density=float(rng.choice([0.01, 0.05, 0.3])), format="csr",
                            random_state=int(rng.integers(1 << 30))).astype(np.float32)
        elif kind == "skewed":
            deg = np.minimum((rng.pareto(1.0, n_rows) * 3).astype(np.int64), n_cols)
            if rng.random() < 0.5 and n_cols >= 1200 - 400:
                deg[int(rng.integers(n_rows))] = min(n_cols, 1500)
            adj = graphgen._csr_from_degrees(deg, n_cols, seed=int(rng.integers(1 << 30)))
        else:
            adj = sp.random(n_rows, n_cols, density=0.002, format="csr",
                            random_state=int(rng.integers(1 << 30))).astype(np.float32)
        unit = bool(rng.random() < 0.4)
        if unit:
            adj.data[:] = 1.0
        else:
            adj.data = (rng.random(adj.nnz, dtype=np.float32) * 4 - 2).astype(np.float32)
        x = (rng.random((n_cols, d), dtype=np.float32) * 2 - 1).astype(np.float32)
        y = (rng.random((n_rows, d), dtype=np.float32) * 2 - 1).astype(np.float32)
        tile = int(rng.choice([0, 0, 4, 16, 32, 64, 128]))
        threshold = int(rng.choice([0, 0, 1, 64, 700, 2 ** 31 - 1, -1, -8]))
        tag = "seed=%d %dx%d nnz=%d d=%d %s unit=%s tile=%d thr=%d" % (seed, n_rows, n_cols, adj.nnz, d, kind, unit,
                                                                   tile, threshold)
        want = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
        got = G.spmm_csr(adj.indptr, adj.indices, None if unit else adj.data, x, feat_tile=tile,
                         long_row_threshold=threshold, use_schedule=bool(rng.random() < 0.85))
        np.testing.assert_array_equal(got, want, err_msg=tag)
        if rng.random() < 0.4:
            parts = int(rng.integers(1, 6))
            s1_pos, s1_idx, vals = util_convert_csr_to_dds(adj, parts)
            np.testing.assert_array_equal(
                G.spmm_dds(s1_pos, s1_idx, vals, x, n_rows, parts, indptr_for_schedule=adj.indptr, feat_tile=tile),
                oracle.spmm_dds(s1_pos, s1_idx, vals, x, n_rows, parts), err_msg=tag)
        coo = adj.tocoo()
        row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
        sorted_rows = 1
        if rng.random() < 0.4 and len(row) > 1:
            perm = rng.permutation(len(row))
            row, col = row[perm], col[perm]
            sorted_rows = 0
        want_e = oracle.sddmm(row, col, x, y)
        stile = int(rng.choice([0, 0, 32, 64, 128]))
        np.testing.assert_allclose(G.sddmm(row, col, x, y, rows_sorted=sorted_rows, feat_tile=stile), want_e, rtol=RTOL,
                                   atol=ATOL, err_msg=tag)
        np.testing.assert_array_equal(G.sddmm_exact(row, col, x, y), want_e, err_msg=tag)
