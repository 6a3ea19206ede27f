"""The fused aggregate-then-score step (fg_spmm_sddmm_fused_f32) against the CPU oracle's two steps:
H = A.X bit for bit, out[e] = dot(H[row e], Y[col e]) within the SDDMM tolerance (scaled by the size of
the products where H's entries are large), and against the two-call GPU result."""
import numpy as np
import pytest
import torch

from conftest import ATOL, RTOL
from featgraph import placeholder

pytestmark = pytest.mark.gpu


def _check(oracle, adj, x, y, h, scores, unit_scale):
    want_h = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
    np.testing.assert_array_equal(h, want_h)
    coo = adj.tocoo()
    want = oracle.sddmm(coo.row, coo.col, y, want_h)  # column side y, row side H
    if unit_scale:
        np.testing.assert_allclose(scores, want, rtol=RTOL, atol=ATOL)
        return
    d = x.shape[1]
    bound = (np.abs(y[coo.col]).astype(np.float64) * np.abs(want_h[coo.row])).sum(-1)
    err = np.abs(scores.astype(np.float64) - want)
    limit = RTOL * np.abs(want) + 2.0 * d * 2.0 ** -24 * bound + 1e-30
    assert np.all(err <= limit), "worst excess %.3g" % float((err - limit).max())


@pytest.mark.parametrize("d", [4, 8, 36, 64, 100, 128])
@pytest.mark.parametrize("threshold", [0, 64, -64, 2 ** 31 - 1])
def test_fused_step_matches_the_two_steps(oracle, d, threshold):
    """Every lane-group width, with the long-row machinery forced on (64: rows of 64+ nonzeros take the ring
    kernels, 1024+ the heavy-row kernel; negative: its 8-warp form) and off, weighted and unweighted."""
    from featgraph_b200 import graphgen
    from featgraph_b200.module.fused import AggregateThenScore
    adj = graphgen.power_law_graph(700, 700 * 60, seed=900 + d, kmax=690).tolil()
    adj[3, :] = 0  # an empty row
    adj = adj.tocsr()
    adj.eliminate_zeros()
    adj.sort_indices()
    n = adj.shape[0]
    x = graphgen.uniform_features((n, d), seed=1)
    y = graphgen.uniform_features((n, d), seed=2)
    for weighted in (False, True):
        a = adj.copy()
        if weighted:
            a.data = graphgen.uniform_features((a.nnz,), seed=3)
        m = AggregateThenScore(a, long_row_threshold=threshold)
        m.build([placeholder((n, d)), placeholder((n, d))])
        for _ in range(2):  # twice: outputs are reused
            h, s = m.run([torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()])
        _check(oracle, a, x, y, h.cpu().numpy(), s.cpu().numpy(), unit_scale=False)


def test_fused_step_equals_the_two_gpu_calls(oracle):
    from featgraph.module import VanillaSDDMMcuda, VanillaSpMMcuda
    from featgraph_b200 import graphgen
    from featgraph_b200.module.fused import AggregateThenScore
    adj = graphgen.rmat_graph(12, 16, seed=77)
    n, d = adj.shape[0], 128
    x = torch.from_numpy(graphgen.uniform_features((n, d), seed=4)).cuda()
    y = torch.from_numpy(graphgen.uniform_features((n, d), seed=5)).cuda()
    m = AggregateThenScore(adj)
    m.build([placeholder((n, d)), placeholder((n, d))])
    h, s = m.run([x, y])
    sp = VanillaSpMMcuda(adj)
    sp.build([placeholder((n, d))], {}, {})
    h2 = sp.run([x])
    assert torch.equal(h, h2)
    sd = VanillaSDDMMcuda(adj.tocoo())
    sd.build([placeholder((n, d)), placeholder((n, d))], {}, {})
    s2 = sd.run([y, h2])
    scale = float(s2.abs().max())
    np.testing.assert_allclose(s.cpu().numpy(), s2.cpu().numpy(), rtol=1e-4, atol=1e-5 * scale)
    assert m.measure_average_time([x, y], 2) > 0


def test_fused_step_argument_errors():
    from featgraph_b200 import graphgen
    from featgraph_b200.module.fused import AggregateThenScore
    adj = graphgen.fixed_degree_graph(50, 5, seed=1)
    m = AggregateThenScore(adj)
    with pytest.raises(ValueError):
        m.build([placeholder((50, 256)), placeholder((50, 256))])
    with pytest.raises(ValueError):
        m.build([placeholder((50, 6)), placeholder((50, 6))])
    with pytest.raises(ValueError):
        m.build([placeholder((50, 8)), placeholder((49, 8))])
    with pytest.raises(RuntimeError):
        m.run([None, None])
