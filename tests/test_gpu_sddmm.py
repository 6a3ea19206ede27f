"""SDDMM on the GPU, through the C ABI, against the CPU oracle, within rtol 1e-5 / atol 1e-4
(the kernel sums a dot product as a tree, the oracle in ascending k)."""
import numpy as np
import pytest
import scipy.sparse as sp

from conftest import ATOL, RTOL

pytestmark = pytest.mark.gpu


def _feat(m, d, seed):
    return (np.random.default_rng(seed).random((m, d), dtype=np.float32) * 2 - 1).astype(np.float32)


def test_reference_test_shape_fixture(oracle, numeric_golden):
    import gpu_util as G
    g = numeric_golden
    out = G.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"])
    np.testing.assert_allclose(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"]), rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(g["sddmm_numpy"], out, rtol=1e-4, atol=1e-4)  # the reference's own check


def test_against_the_references_own_definition_compiled_by_tvm():
    """GPU results against outputs of the reference's SDDMM definition run through a TVM build
    (tests/golden/sddmm_reference_tvm.npz), at the stated tolerance."""
    import gpu_util as G
    from conftest import sddmm_reference_cases
    for name, row, col, src, dst, nfp, ref_out in sddmm_reference_cases():
        for tile in (0, 32):
            np.testing.assert_allclose(G.sddmm(row, col, src, dst, feat_tile=tile), ref_out, rtol=RTOL, atol=ATOL,
                                       err_msg=name)


@pytest.mark.parametrize("d", [1, 3, 4, 8, 20, 32, 33, 48, 64, 100, 128, 200, 256, 384, 512, 640])
@pytest.mark.parametrize("order", ["csr", "shuffled"])
def test_feature_lengths_and_edge_orders(oracle, d, order):
    import gpu_util as G
    coo = sp.random(127, 255, density=0.1, format="csr", random_state=d).tocoo()
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    if order == "shuffled":
        perm = np.random.default_rng(d).permutation(len(row))
        row, col = row[perm], col[perm]
    src, dst = _feat(255, d, 1), _feat(127, d, 2)
    want = oracle.sddmm(row, col, src, dst)
    np.testing.assert_allclose(G.sddmm(row, col, src, dst, rows_sorted=0), want, rtol=RTOL, atol=ATOL)
    if order == "csr":
        np.testing.assert_allclose(G.sddmm(row, col, src, dst, rows_sorted=1), want, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("d,tile", [(128, 32), (128, 64), (100, 32), (256, 64), (512, 128), (96, 64), (640, 0)])
def test_feature_tiles_accumulate_to_the_same_dot_product(oracle, d, tile):
    import gpu_util as G
    coo = sp.random(200, 150, density=0.1, format="csr", random_state=d + tile).tocoo()
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    src, dst = _feat(150, d, 3), _feat(200, d, 4)
    want = oracle.sddmm(row, col, src, dst)
    for s in (0, 1):
        np.testing.assert_allclose(G.sddmm(row, col, src, dst, rows_sorted=s, feat_tile=tile), want,
                                   rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("d", [1, 3, 4, 31, 32, 33, 36, 64, 100, 128, 200, 512])
def test_exact_order_kernel_is_bit_identical_to_the_oracle(oracle, d):
    import gpu_util as G
    coo = sp.random(127, 255, density=0.1, format="coo", random_state=d)  # unsorted edge list
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    src, dst = _feat(255, d, 5), _feat(127, d, 6)
    np.testing.assert_array_equal(G.sddmm_exact(row, col, src, dst), oracle.sddmm(row, col, src, dst))
    for nnz in (0, 1, 33, 2049):
        np.testing.assert_array_equal(G.sddmm_exact(row[:nnz], col[:nnz], src, dst),
                                      oracle.sddmm(row[:nnz], col[:nnz], src, dst))


def test_exact_order_kernel_reproduces_the_references_tvm_output_bit_for_bit():
    """The committed outputs of the reference's own SDDMM definition (compiled by a TVM build)."""
    import gpu_util as G
    from conftest import sddmm_reference_cases
    for name, row, col, src, dst, nfp, ref_out in sddmm_reference_cases():
        np.testing.assert_array_equal(G.sddmm_exact(row, col, src, dst), ref_out, err_msg=name)


def test_exact_option_of_the_module(oracle, numeric_golden):
    import torch
    from featgraph import placeholder
    from featgraph.module import VanillaSDDMMcuda
    g = numeric_golden
    coo = sp.coo_matrix((np.ones(len(g["coo_row"]), np.int32), (g["coo_row"], g["coo_col"])), shape=(127, 255))
    m = VanillaSDDMMcuda(coo)
    m.build([placeholder((255, 128)), placeholder((127, 128))], {}, {"exact": True})
    out = m.run([torch.from_numpy(g["x"]).cuda(), torch.from_numpy(g["y"]).cuda()]).cpu().numpy()
    np.testing.assert_array_equal(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"]))


def test_exact_on_small_integers():
    """Integer-valued features make every fp32 operation exact, whatever the summation tree."""
    import gpu_util as G
    rng = np.random.default_rng(4)
    coo = sp.random(90, 70, density=0.2, format="csr", random_state=4).tocoo()
    for d in (32, 128, 512):
        src = rng.integers(-8, 9, size=(70, d)).astype(np.float32)
        dst = rng.integers(-8, 9, size=(90, d)).astype(np.float32)
        want = (src.astype(np.int64)[coo.col] * dst.astype(np.int64)[coo.row]).sum(-1).astype(np.float32)
        for s in (0, 1):
            np.testing.assert_array_equal(G.sddmm(coo.row, coo.col, src, dst, rows_sorted=s), want)


def test_ragged_edge_counts_and_empty(oracle):
    import gpu_util as G
    src, dst = _feat(40, 64, 1), _feat(30, 64, 2)
    rng = np.random.default_rng(0)
    for nnz in (0, 1, 31, 32, 33, 255, 256, 257, 2049):
        row = np.sort(rng.integers(0, 30, size=nnz)).astype(np.int32)
        col = rng.integers(0, 40, size=nnz).astype(np.int32)
        out = G.sddmm(row, col, src, dst, rows_sorted=1)
        assert out.shape == (nnz,)
        np.testing.assert_allclose(out, oracle.sddmm(row, col, src, dst), rtol=RTOL, atol=ATOL)


def test_long_rows_in_csr_order(oracle):
    import gpu_util as G
    from featgraph_b200 import graphgen
    deg = np.full(20, 3, dtype=np.int64)
    deg[7] = 20000
    a = graphgen._csr_from_degrees(deg, 25000, seed=5).tocoo()
    src = graphgen.uniform_features((25000, 128), seed=6)
    dst = graphgen.uniform_features((20, 128), seed=7)
    np.testing.assert_allclose(G.sddmm(a.row, a.col, src, dst, rows_sorted=1),
                               oracle.sddmm(a.row, a.col, src, dst), rtol=RTOL, atol=ATOL)


def test_2d_partition_order_and_edge_mapping(oracle, numeric_golden):
    import gpu_util as G
    from featgraph_b200.util import util_partition_adj_coo_2d
    g = numeric_golden
    coo = sp.coo_matrix((np.ones(len(g["coo_row"]), np.int32), (g["coo_row"], g["coo_col"])), shape=(127, 255))
    ids, r, c = util_partition_adj_coo_2d(coo, 4, 4)
    out = G.sddmm(r, c, g["x"], g["y"])[np.argsort(ids)]
    np.testing.assert_allclose(out, oracle.sddmm(g["coo_row"], g["coo_col"], g["x"], g["y"]), rtol=RTOL, atol=ATOL)


def test_workload_c1_full_size(oracle):
    """100,000 nodes, 32 neighbours per row, d = 128: 3.2 M edges."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    a = graphgen.workload_graph("C1").tocoo()
    src = graphgen.workload_features("C1", 100_000, 128, 0)
    dst = graphgen.workload_features("C1", 100_000, 128, 1)
    want = oracle.sddmm(a.row, a.col, src, dst, threads=8)
    np.testing.assert_allclose(G.sddmm(a.row, a.col, src, dst, rows_sorted=1), want, rtol=RTOL, atol=ATOL)


def test_coo_validate_reports_order_and_range():
    import ctypes
    import gpu_util as G
    from featgraph_b200 import _native
    L = _native.lib()
    flag = ctypes.c_int32(-1)
    r, c = G.dev(np.array([0, 0, 1, 2], np.int32)), G.dev(np.array([3, 1, 0, 2], np.int32))
    assert L.fg_coo_validate(G.p(r), G.p(c), 3, 4, 4, ctypes.byref(flag), G.stream()) == 0 and flag.value == 1
    r2 = G.dev(np.array([0, 2, 1, 2], np.int32))
    assert L.fg_coo_validate(G.p(r2), G.p(c), 3, 4, 4, ctypes.byref(flag), G.stream()) == 0 and flag.value == 0
    assert L.fg_coo_validate(G.p(r2), G.p(c), 2, 4, 4, ctypes.byref(flag), G.stream()) == 4


# ---- one pass over column blocks (fg_sddmm_coo_f32_planned) ------------------------------------

@pytest.mark.parametrize("d", [4, 36, 64, 128, 132, 200, 256, 384, 500, 512])
@pytest.mark.parametrize("parts", [1, 2, 3, 7])
def test_column_block_plan_gives_the_same_dot_products(oracle, d, parts):
    """Every edge is visited once, in block-major order, and lands at its own place in the caller's edge
    order: rows of very different lengths (empty ones, single edges, runs longer than one 32-edge batch),
    a column count that the block count does not divide."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    adj = graphgen.power_law_graph(301, 301 * 40, seed=300 + parts, kmax=290).tolil()
    adj[7, :] = 0
    adj[300, :] = 0
    adj = adj.tocsr()
    adj.eliminate_zeros()
    adj.sort_indices()
    coo = adj.tocoo()
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    src, dst = _feat(301, d, 11), _feat(301, d, 12)
    want = oracle.sddmm(row, col, src, dst)
    np.testing.assert_allclose(G.sddmm_planned(row, col, src, dst, parts), want, rtol=RTOL, atol=ATOL)


def test_column_block_plan_is_exact_on_integer_valued_features():
    """With small integer features every product and partial sum is exact, so any summation tree must give
    the same bits as numpy: a test of WHICH edges and columns are combined, free of rounding."""
    import gpu_util as G
    rng = np.random.default_rng(5)
    coo = sp.random(180, 1000, density=0.08, format="csr", random_state=9).tocoo()  # wide: many column blocks
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    for d in (128, 200, 512):
        src = rng.integers(-4, 5, (1000, d)).astype(np.float32)
        dst = rng.integers(-4, 5, (180, d)).astype(np.float32)
        want = (src[col] * dst[row]).sum(-1)
        for parts in (2, 5, 16):
            np.testing.assert_array_equal(G.sddmm_planned(row, col, src, dst, parts), want)
        # accumulate adds to what out holds
        base = rng.integers(-100, 100, len(row)).astype(np.float32)
        np.testing.assert_array_equal(G.sddmm_planned(row, col, src, dst, 3, accumulate_onto=base), base + want)


def test_column_block_plan_refuses_what_it_cannot_serve():
    import ctypes
    import gpu_util as G
    from featgraph_b200 import _native
    L = _native.lib()
    coo = sp.random(50, 60, density=0.3, format="csr", random_state=3).tocoo()
    row, col = coo.row.astype(np.int32), coo.col.astype(np.int32)
    h = ctypes.c_void_p()
    # columns descending inside rows
    rc = L.fg_sddmm_plan_create(G.p(G.dev(row)), G.p(G.dev(col[::-1].copy())), 50, 60, len(row), 2, G.stream(),
                                ctypes.byref(h))
    assert rc == 1 and b"CSR order" in L.fg_last_error() and not h.value
    # rows not sorted
    perm = np.random.default_rng(0).permutation(len(row))
    rc = L.fg_sddmm_plan_create(G.p(G.dev(row[perm])), G.p(G.dev(col[perm])), 50, 60, len(row), 2, G.stream(),
                                ctypes.byref(h))
    assert rc == 1 and b"CSR order" in L.fg_last_error()
    # a plan of another adjacency, an unsupported feature length
    rr, cc = G.dev(row), G.dev(col)
    plan = G.SddmmPlan(rr, cc, 50, 60, 2)
    src, dst, out = G.dev(_feat(60, 8, 1)), G.dev(_feat(50, 8, 2)), G.dev(np.zeros(len(row), np.float32))
    rc = L.fg_sddmm_coo_f32_planned(plan.h, G.p(cc), G.p(src), 0, G.p(dst), 0, G.p(out), 50, 60, len(row) - 1, 8, 0,
                                    G.stream())
    assert rc == 1 and b"rebuild the plan" in L.fg_last_error()
    rc = L.fg_sddmm_coo_f32_planned(plan.h, G.p(cc), G.p(src), 0, G.p(dst), 0, G.p(out), 50, 60, len(row), 6, 0,
                                    G.stream())
    assert rc == 1 and b"multiples of 4" in L.fg_last_error()
    plan.close()
    # where the plain call is the better one, the library says so
    assert L.fg_sddmm_auto_partitions(1000, 1000, 50_000, 64) == 1          # fits L2
    assert L.fg_sddmm_auto_partitions(1 << 22, 1 << 22, 1 << 27, 128) == 1  # rows far too short per block
    assert L.fg_sddmm_auto_partitions(232_965, 232_965, 114_615_892, 512) >= 4
