"""The CPU oracle against the fixtures and against itself (no GPU needed)."""
import numpy as np
import scipy.sparse as sp

from featgraph_b200.util import util_convert_csr_to_dds, util_partition_adj_coo_2d


def test_spmm_oracle_vs_scipy_fixture(oracle, numeric_golden):
    g = numeric_golden
    out = oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"])
    # the reference's own bar (tests/test_module_spmm.py:30)
    np.testing.assert_allclose(g["spmm_scipy"], out, rtol=1e-4, atol=1e-4)
    # scipy's CSR kernel also sums in storage order with separate mul and add
    np.testing.assert_array_equal(g["spmm_scipy"], out)


def test_spmm_oracle_layout_knobs_do_not_change_values(oracle, numeric_golden):
    g = numeric_golden
    base = oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"])
    for nfp in (1, 4, 8):
        for copies in (False, True):
            out = oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"],
                                  num_feat_partitions=nfp, with_copies=copies)
            np.testing.assert_array_equal(base, out)
    np.testing.assert_array_equal(
        base, oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"], dynamic=True))


def test_spmm_dds_oracle(oracle, numeric_golden):
    g = numeric_golden
    n, m = 127, 255
    csr = sp.csr_matrix((g["csr_data"], g["csr_indices"], g["csr_indptr"]), shape=(n, m))
    base = oracle.spmm_csr(csr.indptr, csr.indices, csr.data, g["x"])
    one = oracle.spmm_dds(*util_convert_csr_to_dds(csr, 1), g["x"], n, 1)
    np.testing.assert_array_equal(base, one)
    for P, nfp in ((4, 1), (4, 4), (7, 2)):
        out = oracle.spmm_dds(*util_convert_csr_to_dds(csr, P), g["x"], n, P, num_feat_partitions=nfp)
        np.testing.assert_allclose(g["spmm_scipy"], out, rtol=1e-4, atol=1e-4)
    # DDS association differs from CSR association: equal within rounding, not bit for bit
    four = oracle.spmm_dds(*util_convert_csr_to_dds(csr, 4), g["x"], n, 4)
    assert np.abs(four - base).max() < 1e-4


def test_sddmm_oracle_vs_numpy_fixture(oracle, numeric_golden):
    g = numeric_golden
    out = oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"])
    # the reference's own bar (tests/test_module_sddmm.py:37)
    np.testing.assert_allclose(g["sddmm_numpy"], out, rtol=1e-4, atol=1e-4)
    for nfp in (4, 8):
        np.testing.assert_array_equal(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"],
                                                        num_feat_partitions=nfp))
    np.testing.assert_array_equal(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"], threads=4))


def test_spmm_oracle_equals_the_references_own_definitions_compiled_by_tvm(oracle):
    """The pin for SpMM: the reference's CSR (x86 and CUDA) and DDS compute definitions
    (op/vanilla_spmm.py:6-62, 83-125, 149-224), compiled by a TVM build, give exactly the oracle's bits
    on random non-unit values - with separate product and sum roundings, not with fused ones."""
    from conftest import spmm_reference_cases
    n = 0
    for name, kind, adj, x, nfp, ncp, ref_out in spmm_reference_cases():
        if kind == "dds_x86":
            dds = util_convert_csr_to_dds(adj, ncp)
            got = oracle.spmm_dds(*dds, x, adj.shape[0], ncp, num_feat_partitions=nfp)
            fused = oracle.spmm_dds(*dds, x, adj.shape[0], ncp, num_feat_partitions=nfp, use_fma=True)
        else:
            got = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x, num_feat_partitions=nfp, with_copies=True)
            fused = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x, use_fma=True)
        np.testing.assert_array_equal(got, ref_out, err_msg=name)
        assert not np.array_equal(fused, ref_out), name
        n += 1
    assert n == 7


def test_sddmm_oracle_equals_the_references_own_definition_compiled_by_tvm(oracle):
    """The pin for SDDMM: the reference's compute definition (op/vanilla_sddmm.py:6-63), lowered and
    compiled by a TVM build, gives exactly the oracle's bits - with separate product and sum
    roundings, not with fused ones."""
    from conftest import sddmm_reference_cases
    n = 0
    for name, row, col, src, dst, nfp, ref_out in sddmm_reference_cases():
        got = oracle.sddmm(row, col, src, dst, num_feat_partitions=nfp)
        np.testing.assert_array_equal(got, ref_out, err_msg=name)
        assert not np.array_equal(oracle.sddmm(row, col, src, dst, use_fma=True), ref_out), name
        n += 1
    assert n == 4


def test_sddmm_oracle_with_2d_partition(oracle, numeric_golden):
    g = numeric_golden
    coo = sp.coo_matrix((np.ones(len(g["coo_row"]), np.int32), (g["coo_row"], g["coo_col"])), shape=(127, 255))
    ids, r, c = util_partition_adj_coo_2d(coo, 4, 4)
    out = oracle.sddmm(r, c, g["x"], g["y"])[np.argsort(ids)]
    np.testing.assert_array_equal(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"]))


def test_oracle_exact_on_small_integers(oracle):
    """Integer-valued inputs make every fp32 operation exact: compare with int64 arithmetic."""
    rng = np.random.default_rng(5)
    n, m, d = 40, 60, 12
    csr = sp.random(n, m, density=0.2, format="csr", random_state=11)
    csr.data = rng.integers(-4, 5, size=csr.nnz).astype(np.float32)
    csr = csr.astype(np.float32)
    x = rng.integers(-8, 9, size=(m, d)).astype(np.float32)
    y = rng.integers(-8, 9, size=(n, d)).astype(np.float32)
    want = (csr.astype(np.int64) @ x.astype(np.int64)).astype(np.float32)
    np.testing.assert_array_equal(want, oracle.spmm_csr(csr.indptr, csr.indices, csr.data, x))
    np.testing.assert_array_equal(want, oracle.spmm_csr(csr.indptr, csr.indices, csr.data, x, use_fma=True))
    coo = csr.tocoo()
    want_e = (x.astype(np.int64)[coo.col] * y.astype(np.int64)[coo.row]).sum(-1).astype(np.float32)
    np.testing.assert_array_equal(want_e, oracle.sddmm(coo.row, coo.col, x, y))


def test_oracle_fma_switch_is_a_different_rounding(oracle, numeric_golden):
    g = numeric_golden
    rng = np.random.default_rng(9)
    vals = rng.random(len(g["csr_data"]), dtype=np.float32) + 0.5
    a = oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], vals, g["x"], use_fma=False)
    b = oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], vals, g["x"], use_fma=True)
    assert not np.array_equal(a, b)
    np.testing.assert_allclose(a, b, rtol=1e-5, atol=1e-5)


def test_oracle_empty_inputs(oracle):
    out = oracle.spmm_csr(np.zeros(4, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32),
                          np.ones((5, 8), np.float32))
    np.testing.assert_array_equal(out, np.zeros((3, 8), np.float32))
    e = oracle.sddmm(np.zeros(0, np.int32), np.zeros(0, np.int32), np.ones((5, 8), np.float32),
                     np.ones((3, 8), np.float32))
    assert e.shape == (0,)
