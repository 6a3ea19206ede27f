"""The allocation-free SpMM entry point (fg_spmm_csr_f32_static), through the C ABI.

Some callers of this library cannot let it allocate: a serving process whose own pool has taken
all device memory, or a loop that must not run into the device-wide synchronisation hidden in
cudaMalloc.  For them the library rebuilds the row order inside a fixed device array on every
call.  This test checks that the result equals the regular entry point's bit for bit, on two calls
in a row that share that array (a large graph first, then a smaller one with a different degree
mix, so stale contents from the first call would show), and that oversize inputs are refused.

Collected last on purpose (file name), so that a run stopping at the first failure has already
run everything else.
"""
import ctypes

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _run_both(adj, x, feat_tile=0, unit_values=False):
    import torch
    import gpu_util as G
    from featgraph_b200 import _native
    L = _native.lib()
    n_rows, n_cols = adj.shape
    d = x.shape[1]
    ip, ix, xx = G.dev(adj.indptr, np.int32), G.dev(adj.indices, np.int32), G.dev(x)
    vv = None if unit_values else G.dev(adj.data, np.float32)  # None: no value array (all ones)
    # regular path: row schedule object + fg_spmm_csr_f32
    sch = G.Schedule(ip, n_rows)
    buf_a, out_a = G.guarded(n_rows * d)
    _native.check(L.fg_spmm_csr_f32(sch.h, G.p(ip), G.p(ix), G.p(vv), G.p(xx), 0, G.p(out_a), 0, n_rows, n_cols,
                                    adj.nnz, d, feat_tile, G.stream()))
    # allocation-free path: inputs and outputs only
    buf_b, out_b = G.guarded(n_rows * d)
    _native.check(L.fg_spmm_csr_f32_static(G.p(ip), G.p(ix), G.p(vv), G.p(xx), G.p(out_b), n_rows, n_cols,
                                           adj.nnz, d, feat_tile, G.stream()))
    torch.cuda.synchronize()
    assert G.guards_intact(buf_a) and G.guards_intact(buf_b)
    sch.close()
    return out_a.cpu().numpy().reshape(n_rows, d), out_b.cpu().numpy().reshape(n_rows, d)


def test_static_entry_point_matches_regular_one_on_two_calls_in_a_row(oracle):
    from featgraph_b200 import graphgen
    # call 1: power-law graph with long rows, d = 64
    a1 = graphgen.power_law_graph(20_000, 1_500_000, seed=41, kmax=6000)
    a1.data = (np.random.default_rng(42).random(a1.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    x1 = graphgen.uniform_features((20_000, 64), seed=43)
    ref1, got1 = _run_both(a1, x1)
    np.testing.assert_array_equal(got1, ref1)
    np.testing.assert_array_equal(got1, oracle.spmm_csr(a1.indptr, a1.indices, a1.data, x1))
    # call 2 right after, smaller, other degree mix (fixed degree plus empty rows), other d
    a2 = graphgen.fixed_degree_graph(777, 20, seed=44, n_cols=900)
    a2 = a2.tolil()
    a2[5, :] = 0
    a2[600, :] = 0
    a2 = a2.tocsr()
    a2.eliminate_zeros()
    a2 = a2.astype(np.float32)
    x2 = graphgen.uniform_features((900, 36), seed=45)
    ref2, got2 = _run_both(a2, x2)
    np.testing.assert_array_equal(got2, ref2)
    np.testing.assert_array_equal(got2, oracle.spmm_csr(a2.indptr, a2.indices, a2.data, x2))
    # and the first one again: the shared array carries nothing over
    ref3, got3 = _run_both(a1, x1, feat_tile=32)
    np.testing.assert_array_equal(got3, ref1)


def test_static_entry_point_other_kernel_forms(oracle):
    """The forms the first test does not reach: a feature length that is no multiple of 4 (scalar
    kernel), no value array, and a matrix with so many columns that no slice of x can stay in L2 (where
    the regular entry point spreads its kernels over internal streams and this one must not)."""
    from featgraph_b200 import graphgen
    a = graphgen.power_law_graph(3000, 90_000, seed=51, kmax=900)
    x = graphgen.uniform_features((3000, 30), seed=52)
    ref, got = _run_both(a, x)
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(got, oracle.spmm_csr(a.indptr, a.indices, a.data, x))
    ref, got = _run_both(a, x, unit_values=True)
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(got, oracle.spmm_csr(a.indptr, a.indices, np.ones_like(a.data), x))
    wide = graphgen.fixed_degree_graph(2000, 40, seed=53, n_cols=1_200_000)
    xw = graphgen.uniform_features((1_200_000, 8), seed=54)
    ref, got = _run_both(wide, xw)
    np.testing.assert_array_equal(got, ref)
    np.testing.assert_array_equal(got, oracle.spmm_csr(wide.indptr, wide.indices, wide.data, xw))


def test_static_entry_point_allocates_no_device_memory():
    """What the entry point exists for: after one warm-up call (which loads the kernels and looks up the
    scratch array's address), a call must leave the device's free memory exactly as it found it."""
    import torch
    import gpu_util as G
    from featgraph_b200 import _native, graphgen
    L = _native.lib()
    a = graphgen.power_law_graph(20_000, 1_500_000, seed=41, kmax=6000)
    x = graphgen.uniform_features((20_000, 64), seed=43)
    n = a.shape[0]
    ip, ix, xx = G.dev(a.indptr, np.int32), G.dev(a.indices, np.int32), G.dev(x)
    out = torch.empty(n * 64, device="cuda")

    def call():
        _native.check(L.fg_spmm_csr_f32_static(G.p(ip), G.p(ix), None, G.p(xx), G.p(out), n, n, a.nnz, 64, 0,
                                               G.stream()))
        torch.cuda.synchronize()

    call()  # warm-up
    free_before, _ = torch.cuda.mem_get_info()
    call()
    call()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before, "free device memory changed by %d bytes" % (free_before - free_after)


def test_static_entry_point_refuses_more_rows_than_its_array_holds():
    from featgraph_b200 import _native
    L = _native.lib()
    too_many = 1048576 + 1
    rc = L.fg_spmm_csr_f32_static(None, None, None, None, None, too_many, 10, 0, 8, 0, None)
    assert rc == 1
    msg = L.fg_last_error().decode()
    assert "1048576" in msg and "static scratch" in msg
    assert L.fg_spmm_csr_f32_static(None, None, None, None, None, 0, 10, 0, 8, 0, None) == 0
