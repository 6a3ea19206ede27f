"""Backward passes of SpMM / SDDMM (``featgraph_b200.module.autograd.GraphOps``) against torch's own autograd on
the dense formulation of the same ops: fp32 both sides, so agreement is to rounding (rtol 1e-4 / atol 1e-4 on
values of order 1-10), not bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _graph(n_rows, n_cols, seed):
    import scipy.sparse as sp
    a = sp.random(n_rows, n_cols, density=0.08, format="csr", random_state=seed).astype(np.float32)
    a.data[:] = 1.0
    a.sort_indices()
    return a


@pytest.mark.parametrize("d", [4, 20, 64, 200])
def test_spmm_gradients_match_the_dense_formulation(d):
    from featgraph_b200.module.autograd import GraphOps
    adj = _graph(150, 230, 1)
    coo = adj.tocoo()
    row = torch.from_numpy(coo.row.astype(np.int64)).cuda()
    col = torch.from_numpy(coo.col.astype(np.int64)).cuda()
    g = torch.Generator(device="cuda").manual_seed(d)
    x = torch.rand((230, d), device="cuda", generator=g) * 2 - 1
    w = torch.rand((adj.nnz,), device="cuda", generator=g) * 2 - 1
    r = torch.rand((150, d), device="cuda", generator=g)
    ops = GraphOps(adj)
    for weighted in (False, True):
        x1 = x.clone().requires_grad_(True)
        w1 = w.clone().requires_grad_(True) if weighted else None
        out = ops.spmm(x1, w1)
        (out * r).sum().backward()
        x2 = x.clone().requires_grad_(True)
        w2 = w.clone().requires_grad_(True)
        dense = torch.zeros((150, 230), device="cuda").index_put((row, col), w2 if weighted else torch.ones_like(w2))
        want = dense @ x2
        (want * r).sum().backward()
        torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-4)
        torch.testing.assert_close(x1.grad, x2.grad, rtol=1e-4, atol=1e-4)
        if weighted:
            torch.testing.assert_close(w1.grad, w2.grad, rtol=1e-4, atol=1e-4)
    # the gradient is reproducible bit for bit (sequential sums, no atomics)
    x3 = x.clone().requires_grad_(True)
    (ops.spmm(x3, w) * r).sum().backward()
    x4 = x.clone().requires_grad_(True)
    (ops.spmm(x4, w) * r).sum().backward()
    assert torch.equal(x3.grad, x4.grad)


@pytest.mark.parametrize("d", [4, 36, 128])
def test_sddmm_gradients_match_the_dense_formulation(d):
    from featgraph_b200.module.autograd import GraphOps
    adj = _graph(120, 90, 2)
    coo = adj.tocoo()
    row = torch.from_numpy(coo.row.astype(np.int64)).cuda()
    col = torch.from_numpy(coo.col.astype(np.int64)).cuda()
    g = torch.Generator(device="cuda").manual_seed(100 + d)
    src = torch.rand((90, d), device="cuda", generator=g) * 2 - 1
    dst = torch.rand((120, d), device="cuda", generator=g) * 2 - 1
    r = torch.rand((adj.nnz,), device="cuda", generator=g)
    ops = GraphOps(adj)
    s1, t1 = src.clone().requires_grad_(True), dst.clone().requires_grad_(True)
    out = ops.sddmm(s1, t1)
    (out * r).sum().backward()
    s2, t2 = src.clone().requires_grad_(True), dst.clone().requires_grad_(True)
    want = (s2[col] * t2[row]).sum(-1)
    (want * r).sum().backward()
    torch.testing.assert_close(out, want, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(s1.grad, s2.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(t1.grad, t2.grad, rtol=1e-4, atol=1e-4)


def test_one_attention_style_layer_trains_end_to_end():
    """SDDMM scores -> edge weights -> SpMM: gradients flow through both ops into both feature matrices."""
    from featgraph_b200.module.autograd import GraphOps
    adj = _graph(80, 80, 3)
    coo = adj.tocoo()
    row = torch.from_numpy(coo.row.astype(np.int64)).cuda()
    col = torch.from_numpy(coo.col.astype(np.int64)).cuda()
    g = torch.Generator(device="cuda").manual_seed(7)
    q = (torch.rand((80, 16), device="cuda", generator=g) - 0.5).requires_grad_(True)
    v = (torch.rand((80, 16), device="cuda", generator=g) - 0.5).requires_grad_(True)
    ops = GraphOps(adj)
    h = ops.spmm(v, torch.tanh(ops.sddmm(q, q)))
    h.pow(2).sum().backward()
    q2, v2 = q.detach().clone().requires_grad_(True), v.detach().clone().requires_grad_(True)
    score = torch.tanh((q2[col] * q2[row]).sum(-1))
    h2 = torch.zeros((80, 80), device="cuda").index_put((row, col), score) @ v2
    h2.pow(2).sum().backward()
    torch.testing.assert_close(h, h2, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(q.grad, q2.grad, rtol=1e-3, atol=1e-4)
    torch.testing.assert_close(v.grad, v2.grad, rtol=1e-3, atol=1e-4)


@pytest.mark.parametrize("d", [3, 8, 36, 128, 260])
def test_generalized_forms_match_numpy(d):
    """max / min / mean aggregation and the per-edge add / sub / mul against plain numpy (exact: a max, a min
    and one product or sum per element have no rounding freedom; the mean is a sequential sum, then one division)."""
    from featgraph_b200.module.autograd import GraphOps
    adj = _graph(97, 140, 4).tolil()
    adj[11, :] = 0  # a row without nonzeros
    adj = adj.tocsr()
    adj.eliminate_zeros()
    adj.sort_indices()
    coo = adj.tocoo()
    rng = np.random.default_rng(d)
    x = (rng.random((140, d), dtype=np.float32) * 2 - 1).astype(np.float32)
    t = (rng.random((97, d), dtype=np.float32) * 2 - 1).astype(np.float32)
    w = (rng.random(adj.nnz, dtype=np.float32) * 2 - 1).astype(np.float32)
    ops = GraphOps(adj)
    xd, td, wd = torch.from_numpy(x).cuda(), torch.from_numpy(t).cuda(), torch.from_numpy(w).cuda()
    for weight, wn in ((None, np.ones_like(w)), (wd, w)):
        terms = wn[:, None] * x[coo.col]  # one product per (edge, column), rounded once, as on the device
        for name, fn in (("max", np.max), ("min", np.min)):
            want = np.zeros((97, d), dtype=np.float32)
            for r in range(97):
                seg = terms[adj.indptr[r]:adj.indptr[r + 1]]
                if len(seg):
                    want[r] = fn(seg, axis=0)
            np.testing.assert_array_equal(ops.spmm_reduce(xd, name, weight).cpu().numpy(), want)
        want = np.zeros((97, d), dtype=np.float32)
        for r in range(97):
            seg = terms[adj.indptr[r]:adj.indptr[r + 1]]
            acc = np.zeros(d, dtype=np.float32)
            for row_terms in seg:
                acc = (acc + row_terms).astype(np.float32)
            if len(seg):
                want[r] = acc / np.float32(len(seg))
        np.testing.assert_array_equal(ops.spmm_reduce(xd, "mean", weight).cpu().numpy(), want)
    for name, fn in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply)):
        np.testing.assert_array_equal(ops.edge_op(xd, td, name).cpu().numpy(), fn(x[coo.col], t[coo.row]))
