"""Partition utilities: the reference's golden vectors, fixtures made by running the
reference's functions, and a live randomised comparison where the reference is present."""
import numpy as np
import pytest
import scipy.sparse as sp
from hypothesis import given, settings, strategies as st

from conftest import reference_util_or_skip
from featgraph.util import util_convert_csr_to_dds, util_partition_adj_coo_2d
from featgraph_b200.util import nnz_balanced_row_ranges


def _sample_5x5():
    # the matrix of the reference's tests/test_util.py:9-18
    row = np.array([0, 0, 0, 0, 1, 1, 2, 3, 4])
    col = np.array([0, 1, 2, 3, 0, 2, 1, 3, 2])
    ids = np.array([1, 2, 3, 4, 5, 6, 7, 8, 9])
    return sp.coo_matrix((ids, (row, col)), shape=(5, 5), dtype="int32")


def test_dds_known_answer():
    # tests/test_util.py:21-24
    s1_pos, s1_idx, vals = util_convert_csr_to_dds(_sample_5x5().tocsr(), 2)
    np.testing.assert_array_equal(vals, [1, 2, 3, 5, 6, 7, 9, 4, 8])
    np.testing.assert_array_equal(s1_idx, [0, 1, 2, 0, 2, 1, 2, 0, 0])
    np.testing.assert_array_equal(s1_pos, [0, 3, 5, 6, 6, 7, 7, 8, 8, 8, 9, 9])


def test_partition_2d_known_answer():
    # tests/test_util.py:40-43
    coo = _sample_5x5()
    ids, rows, cols = util_partition_adj_coo_2d(coo, 2, 2)
    np.testing.assert_array_equal(ids, [1, 2, 3, 5, 6, 7, 4, 9, 8])
    assert ids.dtype == np.int32
    # the input's data is replaced by 1..nnz, as the reference does
    np.testing.assert_array_equal(coo.data, np.arange(1, 10))
    assert coo.data.dtype == np.int32


def _golden_case(g, i):
    n, m = (int(v) for v in g["c%d_shape" % i])
    csr = sp.csr_matrix((g["c%d_csr_data" % i], g["c%d_csr_indices" % i], g["c%d_csr_indptr" % i]), shape=(n, m))
    coo = sp.coo_matrix((np.ones(len(g["c%d_coo_row" % i]), dtype=np.int32),
                         (g["c%d_coo_row" % i], g["c%d_coo_col" % i])), shape=(n, m))
    return csr, coo


def test_dds_matches_reference_fixtures(partition_golden):
    g = partition_golden
    for i in range(int(g["num_cases"])):
        csr, _ = _golden_case(g, i)
        for P in (1, 2, 3, 4, 7):
            got = util_convert_csr_to_dds(csr, P)
            for name, arr in zip(("pos", "idx", "vals"), got):
                want = g["c%d_dds%d_%s" % (i, P, name)]
                assert arr.dtype == want.dtype
                np.testing.assert_array_equal(arr, want)


def test_partition_2d_matches_reference_fixtures(partition_golden):
    g = partition_golden
    for i in range(int(g["num_cases"])):
        _, coo = _golden_case(g, i)
        for Pr, Pc in ((1, 1), (2, 2), (4, 4), (3, 5), (8, 1)):
            got = util_partition_adj_coo_2d(coo.copy(), Pr, Pc)
            for name, arr in zip(("ids", "row", "col"), got):
                want = g["c%d_p2d%dx%d_%s" % (i, Pr, Pc, name)]
                assert arr.dtype == want.dtype
                np.testing.assert_array_equal(arr, want)


def test_partition_2d_rejects_duplicates():
    coo = sp.coo_matrix((np.ones(3, dtype=np.int32), ([0, 0, 1], [1, 1, 0])), shape=(2, 2))
    with pytest.raises(ValueError):
        util_partition_adj_coo_2d(coo, 2, 2)


@settings(max_examples=60, deadline=None)
@given(st.integers(1, 30), st.integers(1, 30), st.sampled_from([0.0, 0.1, 0.5, 1.0]),
       st.integers(1, 9), st.integers(1, 9), st.integers(0, 2 ** 20), st.booleans())
def test_live_against_reference(n, m, density, p1, p2, seed, shuffle_rows):
    ref = reference_util_or_skip()
    csr = sp.random(n, m, density=density, format="csr", random_state=seed).astype("float32")
    if shuffle_rows:  # storage order inside a row is not always sorted
        rng = np.random.default_rng(seed)
        for r in range(n):
            s, e = csr.indptr[r], csr.indptr[r + 1]
            perm = rng.permutation(e - s)
            csr.indices[s:e] = csr.indices[s:e][perm]
            csr.data[s:e] = csr.data[s:e][perm]
        csr.has_sorted_indices = False
    for a, b in zip(ref.util_convert_csr_to_dds(csr, p1), util_convert_csr_to_dds(csr, p1)):
        assert a.dtype == b.dtype
        np.testing.assert_array_equal(a, b)
    coo = sp.random(n, m, density=density, format="coo", random_state=seed + 1).astype("int32")
    coo2 = coo.copy()
    for a, b in zip(ref.util_partition_adj_coo_2d(coo, p1, p2), util_partition_adj_coo_2d(coo2, p1, p2)):
        assert a.dtype == b.dtype
        np.testing.assert_array_equal(a, b)
    np.testing.assert_array_equal(coo.data, coo2.data)


@settings(max_examples=40, deadline=None)
@given(st.integers(1, 40), st.integers(1, 40), st.integers(1, 8), st.integers(0, 2 ** 20))
def test_dds_is_a_regrouping(n, m, P, seed):
    """Every nonzero appears once, in its column block, with its value."""
    csr = sp.random(n, m, density=0.3, format="csr", random_state=seed).astype("float32")
    s1_pos, s1_idx, vals = util_convert_csr_to_dds(csr, P)
    w = -(-m // P)
    rebuilt = sp.lil_matrix((n, m), dtype=np.float32)
    for k in range(P):
        for r in range(n):
            for e in range(s1_pos[k * (n + 1) + r], s1_pos[k * (n + 1) + r + 1]):
                c = s1_idx[e] + k * w
                assert k * w <= c < min((k + 1) * w, m) or (k == P - 1 and c < m)
                rebuilt[r, c] = vals[e]
    assert (rebuilt.tocsr() != csr).nnz == 0
    assert s1_pos[-1] == csr.nnz


def test_nnz_balanced_row_ranges_definition():
    rng = np.random.default_rng(3)
    deg = rng.integers(0, 50, size=1000)
    deg[17] = 5000
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    nnz = int(indptr[-1])
    for P in (1, 2, 3, 4, 8):
        b = nnz_balanced_row_ranges(indptr, P)
        want = np.searchsorted(indptr, [(p * nnz) // P for p in range(P + 1)], side="left")
        want[0], want[-1] = 0, 1000
        np.testing.assert_array_equal(b, want)
        assert b.dtype == np.int64 and np.all(np.diff(b) >= 0)
        shard_nnz = indptr[b[1:]] - indptr[b[:-1]]
        assert shard_nnz.sum() == nnz
        assert shard_nnz.max() <= nnz / P + deg.max()


def test_nnz_balanced_row_ranges_edge_cases():
    np.testing.assert_array_equal(nnz_balanced_row_ranges(np.zeros(1, np.int32), 4), [0, 0, 0, 0, 0])
    np.testing.assert_array_equal(nnz_balanced_row_ranges(np.zeros(6, np.int32), 2), [0, 0, 5])
    b = nnz_balanced_row_ranges(np.array([0, 10], np.int32), 4)
    assert b[0] == 0 and b[-1] == 1 and np.all(np.diff(b) >= 0)
