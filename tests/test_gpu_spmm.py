"""SpMM on the GPU, through the C ABI, against the CPU oracle: bit for bit."""
import numpy as np
import pytest
import scipy.sparse as sp

pytestmark = pytest.mark.gpu


def _rand_csr(n, m, density, seed, ones=False):
    a = sp.random(n, m, density=density, format="csr", random_state=seed).astype(np.float32)
    if ones:
        a.data[:] = 1.0
    else:
        a.data = (np.random.default_rng(seed).random(a.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    return a


def _feat(m, d, seed):
    return (np.random.default_rng(seed).random((m, d), dtype=np.float32) * 2 - 1).astype(np.float32)


def test_reference_test_shape_fixture(oracle, numeric_golden):
    import gpu_util as G
    g = numeric_golden
    out = G.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"])
    np.testing.assert_array_equal(out, oracle.spmm_csr(g["csr_indptr"], g["csr_indices"], g["csr_data"], g["x"]))
    np.testing.assert_allclose(g["spmm_scipy"], out, rtol=1e-4, atol=1e-4)  # the reference's own check


def test_bit_identical_to_the_references_own_definitions_compiled_by_tvm():
    """GPU results against the committed outputs of the reference's SpMM definitions run through a TVM
    build (tests/golden/spmm_reference_tvm.npz): CSR and DDS, random non-unit values, bit for bit."""
    import gpu_util as G
    from conftest import spmm_reference_cases
    from featgraph_b200.util import util_convert_csr_to_dds
    for name, kind, adj, x, nfp, ncp, ref_out in spmm_reference_cases():
        if kind == "dds_x86":
            s1_pos, s1_idx, vals = util_convert_csr_to_dds(adj, ncp)
            got = G.spmm_dds(s1_pos, s1_idx, vals, x, adj.shape[0], ncp, indptr_for_schedule=adj.indptr)
        else:
            got = G.spmm_csr(adj.indptr, adj.indices, adj.data, x)
        np.testing.assert_array_equal(got, ref_out, err_msg=name)


@pytest.mark.parametrize("d", [1, 3, 4, 8, 20, 32, 33, 64, 100, 128, 256, 512])
def test_feature_lengths(oracle, d):
    import gpu_util as G
    a = _rand_csr(127, 255, 0.1, seed=d)
    x = _feat(255, d, seed=1000 + d)
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x), want)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x, use_schedule=False), want)


@pytest.mark.parametrize("tile", [4, 8, 16, 32, 64, 128])
@pytest.mark.parametrize("d", [32, 96, 128])
def test_feature_tile_never_changes_values(oracle, d, tile):
    import gpu_util as G
    a = _rand_csr(300, 200, 0.15, seed=7)
    x = _feat(200, d, seed=8)
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x, feat_tile=tile), want)


def test_unfused_rounding_is_the_one_matched(oracle):
    import gpu_util as G
    a = _rand_csr(200, 200, 0.3, seed=21)
    x = _feat(200, 64, seed=22)
    out = G.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(out, oracle.spmm_csr(a.indptr, a.indices, a.data, x, use_fma=False))
    assert not np.array_equal(out, oracle.spmm_csr(a.indptr, a.indices, a.data, x, use_fma=True))


@pytest.mark.parametrize("d", [3, 32, 64, 128])
def test_unit_values_need_no_value_array(oracle, d):
    """vals = NULL means all ones: same values as an explicit all-ones array, long rows included, and
    non-finite / signed-zero features behave as in the oracle."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    deg = np.array([0, 1, 7, 33, 1500, 64, 5000, 2, 31, 32], dtype=np.int64)
    a = graphgen._csr_from_degrees(deg, 7000, seed=11)
    x = graphgen.uniform_features((7000, d), seed=12 + d)
    x[a.indices[0], 0] = -0.0
    x[a.indices[5], d - 1] = np.inf
    x[a.indices[2000], 1 % d] = np.nan
    want = oracle.spmm_csr(a.indptr, a.indices, np.ones(a.nnz, np.float32), x)
    for threshold in (0, 1024, 2 ** 31 - 1):
        got = G.spmm_csr(a.indptr, a.indices, None, x, long_row_threshold=threshold)
        np.testing.assert_array_equal(got, want)  # NaN positions included
        finite = ~np.isnan(want)
        np.testing.assert_array_equal(np.signbit(got[finite]), np.signbit(want[finite]))  # signed zeros too
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, None, x, use_schedule=False), want)


def test_empty_rows_empty_matrix_and_single_row(oracle):
    import gpu_util as G
    # rows 0, 3 and the last are empty
    indptr = np.array([0, 0, 2, 5, 5, 6, 6], dtype=np.int32)
    indices = np.array([1, 3, 0, 2, 3, 1], dtype=np.int32)
    vals = np.arange(1, 7, dtype=np.float32)
    x = _feat(4, 12, seed=3)
    np.testing.assert_array_equal(G.spmm_csr(indptr, indices, vals, x), oracle.spmm_csr(indptr, indices, vals, x))
    # no nonzeros at all: output must be written as zeros
    z = G.spmm_csr(np.zeros(6, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32), x[:4])
    np.testing.assert_array_equal(z, np.zeros((5, 12), np.float32))
    # zero rows: nothing to do, no error
    G.spmm_csr(np.zeros(1, np.int32), np.zeros(0, np.int32), np.zeros(0, np.float32), x, check_guards=True)


def test_one_very_long_row_among_short_ones(oracle):
    """A 20000-nonzero row: sequential fp32 summation order is what makes this bit-exact."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    deg = np.full(64, 5, dtype=np.int64)
    deg[40] = 20000
    deg[3] = 4097
    a = graphgen._csr_from_degrees(deg, 30000, seed=99)
    for d in (4, 32, 128):
        x = graphgen.uniform_features((30000, d), seed=100 + d)
        want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
        np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x), want)


@pytest.mark.parametrize("d", [4, 32, 36, 100, 128, 33])
def test_long_rows_take_the_deep_pipeline_and_stay_exact(oracle, d):
    """Rows of 1024+ nonzeros run in the long-row kernel: lengths around the chunk (8) and ring
    (32) sizes, a mix with short rows, and random (non-unit) values."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    deg = np.array([1024, 1025, 1031, 1032, 1056, 2048, 5000, 1023, 0, 7, 1055, 3001, 1, 1040], dtype=np.int64)
    a = graphgen._csr_from_degrees(deg, 6000, seed=77)
    a.data = (np.random.default_rng(78).random(a.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    x = graphgen.uniform_features((6000, d), seed=79 + d)
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x), want)  # split chosen per launch
    for threshold in (1, 64, 1024, 1031, 4096, 2 ** 31 - 1):
        np.testing.assert_array_equal(
            G.spmm_csr(a.indptr, a.indices, a.data, x, long_row_threshold=threshold), want)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x, feat_tile=32, long_row_threshold=1024), want)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x, use_schedule=False), want)


@pytest.mark.parametrize("d", [4, 32, 36, 100, 128])
@pytest.mark.parametrize("unit", [False, True])
def test_heavy_rows_take_the_block_per_row_kernel_and_stay_exact(oracle, d, unit):
    """With a fixed threshold T, rows of 16 T nonzeros and more go to the kernel in which the warps of
    a block take turns on one row: fewer stages than warps, exact multiples of the 32-nonzero stage,
    one more and one less, a long row, and the ring kernel and the plain kernel beside it."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    deg = np.array([16, 17, 31, 32, 33, 63, 64, 65, 95, 96, 97, 127, 128, 129, 160, 1000, 4099, 0, 3, 15, 256, 20001],
                   dtype=np.int64)
    a = graphgen._csr_from_degrees(deg, 30000, seed=301)
    if not unit:
        a.data = (np.random.default_rng(302).random(a.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    x = graphgen.uniform_features((30000, d), seed=303 + d)
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    for threshold in (1, 2, 8, 64, -1, -4, -64):  # heavy from 16, 32, 128, 1024 nonzeros; < 0: 8 warps per row
        got = G.spmm_csr(a.indptr, a.indices, None if unit else a.data, x, long_row_threshold=threshold)
        np.testing.assert_array_equal(got, want, err_msg="threshold %d" % threshold)


def test_every_row_long(oracle):
    import gpu_util as G
    from featgraph_b200 import graphgen
    a = graphgen._csr_from_degrees(np.full(37, 1500, dtype=np.int64), 4000, seed=5)
    x = graphgen.uniform_features((4000, 64), seed=6)
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x, long_row_threshold=1024), want)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x), want)


def test_unsorted_and_duplicate_columns_keep_storage_order(oracle):
    import gpu_util as G
    rng = np.random.default_rng(5)
    n, m, d = 50, 40, 32
    deg = rng.integers(0, 70, size=n)
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    indices = rng.integers(0, m, size=indptr[-1]).astype(np.int32)  # unsorted, with repeats
    vals = (rng.random(indptr[-1], dtype=np.float32) * 2 - 1).astype(np.float32)
    x = _feat(m, d, seed=6)
    np.testing.assert_array_equal(G.spmm_csr(indptr, indices, vals, x), oracle.spmm_csr(indptr, indices, vals, x))


def test_nan_and_inf_features_stay_in_their_rows(oracle):
    import gpu_util as G
    a = _rand_csr(64, 64, 0.1, seed=31, ones=True)
    x = _feat(64, 32, seed=32)
    x[5, 3] = np.inf
    x[9, 0] = np.nan
    want = oracle.spmm_csr(a.indptr, a.indices, a.data, x)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x), want)  # NaN == NaN here


@pytest.mark.parametrize("parts", [1, 2, 4, 7])
@pytest.mark.parametrize("d", [3, 32, 128])
def test_dds_partitions_match_dds_oracle(oracle, parts, d):
    import gpu_util as G
    from featgraph_b200.util import util_convert_csr_to_dds
    a = _rand_csr(127, 255, 0.1, seed=40 + parts)
    x = _feat(255, d, seed=50 + d)
    s1_pos, s1_idx, vals = util_convert_csr_to_dds(a, parts)
    want = oracle.spmm_dds(s1_pos, s1_idx, vals, x, 127, parts)
    np.testing.assert_array_equal(G.spmm_dds(s1_pos, s1_idx, vals, x, 127, parts), want)
    np.testing.assert_array_equal(
        G.spmm_dds(s1_pos, s1_idx, vals, x, 127, parts, indptr_for_schedule=a.indptr), want)


def test_row_schedule_is_degree_descending_and_stable():
    import torch
    import gpu_util as G
    from featgraph_b200 import _native
    from featgraph_b200.module import _device
    rng = np.random.default_rng(1)
    deg = rng.integers(0, 6, size=5000)
    deg[77] = 900
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    sch = G.Schedule(G.dev(indptr), 5000)
    addr = _native.lib().fg_row_schedule_order(sch.h)
    order = _device.view_device_int32(addr, 5000, torch.device("cuda", torch.cuda.current_device())).cpu().numpy()
    want = np.argsort(-deg, kind="stable")
    np.testing.assert_array_equal(order, want)
    L = _native.lib()
    assert L.fg_row_schedule_rows_at_least(sch.h, 1024) == 0
    assert L.fg_row_schedule_rows_at_least(sch.h, 512) == 1
    sch.close()
    deg[[5, 4000, 77]] = [1024, 3000, 1023]
    indptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int32)
    sch = G.Schedule(G.dev(indptr), 5000, long_row_threshold=1000)
    assert L.fg_row_schedule_rows_at_least(sch.h, 1024) == 2
    assert L.fg_row_schedule_rows_at_least(sch.h, 1000) == 3
    assert L.fg_row_schedule_rows_at_least(sch.h, 64) == int((deg >= 64).sum())
    assert L.fg_row_schedule_rows_at_least(sch.h, 1001) == -1
    assert L.fg_row_schedule_num_rows(sch.h) == 5000
    sch.close()


def test_workload_c0_full_size(oracle):
    """The CPU-runnable configuration: 10,000 nodes, 20 neighbours per row, d = 64."""
    import gpu_util as G
    from featgraph_b200 import graphgen
    a = graphgen.workload_graph("C0")
    x = graphgen.workload_features("C0", 10_000, 64)
    np.testing.assert_array_equal(G.spmm_csr(a.indptr, a.indices, a.data, x),
                                  oracle.spmm_csr(a.indptr, a.indices, a.data, x))


def test_bad_adjacency_is_reported():
    import gpu_util as G
    from featgraph_b200 import _native
    L = _native.lib()
    indptr = G.dev(np.array([0, 2, 1, 3], np.int32))
    indices = G.dev(np.array([0, 1, 9], np.int32))
    assert L.fg_csr_validate(G.p(indptr), G.p(indices), 3, 4, 3, G.stream()) == 4
    good = G.dev(np.array([0, 1, 2, 3], np.int32))
    assert L.fg_csr_validate(G.p(good), G.p(indices), 3, 4, 3, G.stream()) == 4  # column 9 of 4
    assert L.fg_csr_validate(G.p(good), G.p(indices), 3, 10, 3, G.stream()) == 0


def test_schedule_of_another_adjacency_is_refused():
    """The rows kernels take row extents from the schedule's cache: a schedule built from a different
    adjacency (same row count, other nonzero count) must be refused on the host, not run."""
    import torch
    import gpu_util as G
    from featgraph_b200 import _native, graphgen
    a = graphgen.fixed_degree_graph(300, 20, seed=5)
    b = graphgen.fixed_degree_graph(300, 12, seed=6)
    x = G.dev(graphgen.uniform_features((300, 16), seed=7))
    ip_a, ip_b, ix_b = G.dev(a.indptr, np.int32), G.dev(b.indptr, np.int32), G.dev(b.indices, np.int32)
    sch = G.Schedule(ip_a, 300)
    out = torch.zeros(300 * 16, device="cuda")
    L = _native.lib()
    rc = L.fg_spmm_csr_f32(sch.h, G.p(ip_b), G.p(ix_b), None, G.p(x), 0, G.p(out), 0, 300, 300, b.nnz, 16, 0,
                           G.stream())
    assert rc == 1 and b"rebuild the schedule" in L.fg_last_error()
    torch.cuda.synchronize()
    assert not out.any()  # nothing ran
    sch.close()
