"""Host-side logic of the multi-GPU layer on CPU ranks (gloo, world size 2 and 3): row ranges,
local CSR slices and the uneven all-gather of feature rows.  The per-rank compute is done by
the CPU oracle here (the GPU kernels are exercised by the -m gpu tests); what is checked is that
sharding plus gathering reproduces the single-process result bit for bit."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import ROOT


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _worker(rank, world, port, tmpdir):
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from featgraph_b200 import graphgen
        from featgraph_b200.sharded import (all_gather_padded, all_gather_rows, padded_layout,
                                            remap_columns_to_padded, shard_csr_rows)
        from featgraph_b200.util import nnz_balanced_row_ranges

        n, d = 600, 24
        adj = graphgen.power_law_graph(n, 30_000, seed=11, kmax=500)
        x = graphgen.uniform_features((n, d), seed=12)
        y = graphgen.uniform_features((n, d), seed=13)
        bounds = nnz_balanced_row_ranges(adj.indptr, world)
        lo, hi = int(bounds[rank]), int(bounds[rank + 1])

        local = shard_csr_rows(adj, bounds, rank)
        assert local.shape == (hi - lo, n) and local.indptr[0] == 0
        assert local.indptr.dtype == np.int32 and local.indices.dtype == np.int32
        np.testing.assert_array_equal(local.indices, adj.indices[adj.indptr[lo]:adj.indptr[hi]])
        # a rank can also generate its rows alone and get the same slice
        alone = graphgen.power_law_graph(n, 30_000, seed=11, kmax=500, rows=(lo, hi))
        np.testing.assert_array_equal(alone.indices, local.indices)
        np.testing.assert_array_equal(alone.indptr, local.indptr)

        # uneven all-gather of the feature rows
        full = torch.full((n, d), float("nan"))
        all_gather_rows(full, torch.from_numpy(x[lo:hi].copy()), bounds)
        np.testing.assert_array_equal(full.numpy(), x)

        # the same through equal slots of a padded buffer, with column ids remapped into it
        slot, shift = padded_layout(bounds)
        assert slot == int(np.diff(bounds).max())
        padded = torch.zeros((world * slot, d))
        all_gather_padded(padded, torch.from_numpy(x[lo:hi].copy()), bounds)
        for p in range(world):
            np.testing.assert_array_equal(padded[p * slot:p * slot + int(bounds[p + 1] - bounds[p])].numpy(),
                                          x[int(bounds[p]):int(bounds[p + 1])])
        remapped = remap_columns_to_padded(local, bounds)
        assert remapped.shape == (hi - lo, world * slot) and remapped.indices.dtype == np.int32
        np.testing.assert_array_equal(padded.numpy()[remapped.indices], x[local.indices])
        np.testing.assert_array_equal(
            oracle.spmm_csr(remapped.indptr, remapped.indices, remapped.data, padded.numpy()),
            oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)[lo:hi])

        # per-rank SpMM on the gathered features == rows [lo, hi) of the whole product
        whole = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
        mine = oracle.spmm_csr(local.indptr, local.indices, local.data, full.numpy())
        np.testing.assert_array_equal(mine, whole[lo:hi])

        # per-rank SDDMM: edges of the local rows, row-side features local, column-side gathered
        coo = adj.tocoo()
        whole_e = oracle.sddmm(coo.row, coo.col, x, y)
        lc = local.tocoo()
        mine_e = oracle.sddmm(lc.row, lc.col, full.numpy(), y[lo:hi])
        np.testing.assert_array_equal(mine_e, whole_e[adj.indptr[lo]:adj.indptr[hi]])

        # wrong-sized local block is refused before any communication
        with pytest.raises(ValueError):
            all_gather_rows(full, torch.zeros(hi - lo + 1, d), bounds)
        open(os.path.join(tmpdir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_sharding_and_gather_on_cpu_ranks(tmp_path, world):
    import oracle
    oracle.build()  # once, before the ranks race to build it
    from featgraph_b200 import build
    build.build_graphgen()
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok%d" % r for r in range(world)]


def _worker_layouts(rank, world, port, tmpdir):
    """GatheredFeatures picks the padded layout for row blocks of similar size and the plain one for
    very unequal blocks; either way the buffer indexed by the (re)mapped column ids holds x."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import scipy.sparse as sp
        from featgraph_b200.sharded import GatheredFeatures, remap_columns, shard_csr_rows, use_padded_layout
        n, d = 300, 8
        adj = sp.random(n, n, density=0.05, format="csr", random_state=3).astype(np.float32)
        x = np.random.default_rng(4).random((n, d), dtype=np.float32)
        for bounds, padded in ((np.array([0, 140, 300]), True), (np.array([0, 10, 300]), False)):
            assert use_padded_layout(bounds) == padded
            lo, hi = int(bounds[rank]), int(bounds[rank + 1])
            # peer_copy needs NCCL and symmetric memory: on other backends the collective is used
            g = GatheredFeatures(bounds, d, peer_copy=padded)
            assert g.exchange == "all-gather"
            assert g._slot(rank) == ((rank * g.slot, rank * g.slot + hi - lo) if padded else (lo, hi))
            assert g.padded == padded and g.full.shape[0] == (2 * int(np.diff(bounds).max()) if padded else n)
            g.gather(torch.from_numpy(x[lo:hi].copy()))
            local = remap_columns(shard_csr_rows(adj, bounds, rank), bounds)
            assert local.shape == (hi - lo, g.full.shape[0])
            np.testing.assert_array_equal(g.full.numpy()[local.indices], x[adj.indices[adj.indptr[lo]:adj.indptr[hi]]])
            g.gather_async(torch.from_numpy(x[lo:hi].copy())).wait()  # gloo: the blocking path
            np.testing.assert_array_equal(g.full.numpy()[local.indices], x[adj.indices[adj.indptr[lo]:adj.indptr[hi]]])
        open(os.path.join(tmpdir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


def test_gather_layout_follows_the_row_ranges(tmp_path):
    mp.spawn(_worker_layouts, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok0", "ok1"]


def _worker_peer_leaves(rank, world, port, tmpdir):
    """Rank 1 leaves between steps (no collective in flight); rank 0's next exchange must end with an
    ExchangeError within the process group's timeout instead of hanging."""
    import datetime
    import time
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    from featgraph_b200.sharded import ExchangeError, all_gather_padded, padded_layout
    bounds = np.array([0, 5, 9])
    slot, _ = padded_layout(bounds)
    local = torch.full((int(bounds[rank + 1] - bounds[rank]), 4), float(rank))
    padded = torch.zeros((world * slot, 4))
    all_gather_padded(padded, local, bounds)  # step 1: everybody is there
    assert padded[slot, 0] == 1.0 and padded[0, 0] == 0.0
    if rank == 1:
        open(os.path.join(tmpdir, "left"), "w").write("1")
        os._exit(0)  # gone before step 2
    t0 = time.time()
    try:
        all_gather_padded(padded, local, bounds)
    except ExchangeError as exc:
        assert "all-gather failed" in str(exc)
        open(os.path.join(tmpdir, "detected"), "w").write("%.1f" % (time.time() - t0))
    os._exit(0)  # skip the group's teardown: the peer is gone


def test_a_missing_peer_is_reported_not_waited_for_forever(tmp_path):
    ctx = mp.get_context("spawn")
    port = _free_port()
    procs = [ctx.Process(target=_worker_peer_leaves, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=120)
        assert not p.is_alive()
    assert os.path.exists(os.path.join(tmp_path, "left"))
    assert os.path.exists(os.path.join(tmp_path, "detected")), "rank 0 did not see an ExchangeError"
    assert float(open(os.path.join(tmp_path, "detected")).read()) < 60


def _worker_needed_rows(rank, world, port, tmpdir):
    """The needed-rows exchange on a skewed graph: every rank receives exactly the feature rows its shard's
    column ids reference, the remapped shard indexes them, and the per-rank result equals the rows of the
    whole product bit for bit (the remap is increasing, so every sum keeps its order)."""
    sys.path.insert(0, ROOT)
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        import oracle
        from featgraph_b200 import graphgen
        from featgraph_b200.sharded import NeededFeatures, NeededRows, needed_rows_pay, shard_csr_rows
        from featgraph_b200.util import nnz_balanced_row_ranges
        adj = graphgen.rmat_graph(11, 4, seed=5)  # 2048 vertices, a few thousand edges: many untouched columns
        n, d = adj.shape[0], 12
        x = graphgen.uniform_features((n, d), seed=6)
        y = graphgen.uniform_features((n, d), seed=7)
        bounds = nnz_balanced_row_ranges(adj.indptr, world)
        lo, hi = int(bounds[rank]), int(bounds[rank + 1])
        local = shard_csr_rows(adj, bounds, rank)
        rows = NeededRows(local, bounds)
        want_needed = np.unique(local.indices)
        np.testing.assert_array_equal(rows.needed, want_needed)
        assert rows.n_compact == len(want_needed) < n and rows.adj.shape == (hi - lo, len(want_needed))
        assert int(rows.recv_counts.sum()) == len(want_needed)
        assert needed_rows_pay(rows) in (True, False)
        # what this rank sends: for each peer, that peer's needed ids inside [lo, hi), in ascending order
        feats = NeededFeatures(rows, d, peer_pull=True)  # needs NCCL and symmetric memory: here the all-to-all is used
        assert feats.exchange == "all-to-all" and feats.local_input is None
        feats.wait_writable()  # nothing to wait for
        # the request lists the peer-pull form reads with: needed ids as row numbers within their owners' blocks
        owner = np.searchsorted(bounds[1:], rows.needed, side="right")
        np.testing.assert_array_equal(rows.request_rows.numpy(), rows.needed - bounds[owner])
        # ... so that reading owner q's block at its part of the list fills this rank's compact buffer in order
        cut = np.concatenate([[0], np.cumsum(rows.recv_counts)])
        pulled = np.concatenate([x[bounds[q]:bounds[q + 1]][rows.request_rows.numpy()[cut[q]:cut[q + 1]]]
                                 for q in range(world)])
        np.testing.assert_array_equal(pulled, x[rows.needed])
        for _ in range(2):  # twice: buffers are reused
            feats.gather(torch.from_numpy(x[lo:hi].copy()))
            np.testing.assert_array_equal(feats.full.numpy()[:rows.n_compact], x[want_needed])
        np.testing.assert_array_equal(feats.full.numpy()[rows.adj.indices], x[local.indices])
        whole = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
        mine = oracle.spmm_csr(rows.adj.indptr, rows.adj.indices, rows.adj.data, feats.full.numpy())
        np.testing.assert_array_equal(mine, whole[lo:hi])
        coo = adj.tocoo()
        whole_e = oracle.sddmm(coo.row, coo.col, x, y)
        lc = rows.adj.tocoo()
        mine_e = oracle.sddmm(lc.row, lc.col, feats.full.numpy(), y[lo:hi])
        np.testing.assert_array_equal(mine_e, whole_e[adj.indptr[lo]:adj.indptr[hi]])
        feats.gather_async(torch.from_numpy(y[lo:hi].copy())).wait()  # gloo: the blocking path
        np.testing.assert_array_equal(feats.full.numpy()[:rows.n_compact], y[want_needed])
        open(os.path.join(tmpdir, "ok%d" % rank), "w").write("ok")
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_needed_rows_exchange_on_cpu_ranks(tmp_path, world):
    import oracle
    oracle.build()
    from featgraph_b200 import build
    build.build_graphgen()
    mp.spawn(_worker_needed_rows, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    assert sorted(os.listdir(tmp_path)) == ["ok%d" % r for r in range(world)]
