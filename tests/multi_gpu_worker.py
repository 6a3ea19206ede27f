"""One rank of the multi-GPU parity check (launched by test_multi_gpu.py through
torch.distributed.run).  Each rank checks its own shard of SpMM / SDDMM against the CPU oracle, for a
few feature lengths."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    rank = int(os.environ["RANK"])
    local_rank = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    dist.init_process_group("nccl", device_id=device)
    world = dist.get_world_size()
    for graph in ("power-law", "r-mat"):
        check_graph(graph, rank, world, device)
    dist.barrier()
    if rank == 0:
        print("MULTI_GPU_SMALL_OK world=%d" % world, flush=True)
    if os.environ.get("FG_MULTI_GPU_FULL_SIZE", "1") != "0":
        check_full_size_shard(rank, world, device)
        dist.barrier()
        if rank == 0:
            print("MULTI_GPU_FULL_SIZE_OK world=%d" % world, flush=True)
    if rank == 0:
        print("MULTI_GPU_OK world=%d" % world, flush=True)
    dist.destroy_process_group()


def check_graph(graph, rank, world, device):
    import oracle
    from featgraph_b200 import graphgen
    from featgraph_b200.sharded import GatheredFeatures, ShardedSDDMM, ShardedSpMM, shard_csr_rows
    from featgraph_b200.util import nnz_balanced_row_ranges

    if graph == "power-law":  # row blocks of similar size: the padded gather layout
        n = 6000
        adj = graphgen.power_law_graph(n, 600_000, seed=61, kmax=4000)
    else:  # R-MAT: nnz-balanced blocks of very different row counts: the plain layout, uneven all-gather
        adj = graphgen.rmat_graph(13, 32, seed=71)
        n = adj.shape[0]
    bounds = nnz_balanced_row_ranges(adj.indptr, world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    local = shard_csr_rows(adj, bounds, rank)
    spmm = ShardedSpMM(local, bounds, device=device)
    sddmm = ShardedSDDMM(local, bounds, device=device)
    coo = adj.tocoo()
    for d in (32, 256, 200):
        x = graphgen.uniform_features((n, d), seed=62 + d)
        y = graphgen.uniform_features((n, d), seed=63 + d)
        spmm.build(d)
        sddmm.build(d)
        xl = torch.from_numpy(x[lo:hi].copy()).to(device)
        yl = torch.from_numpy(y[lo:hi].copy()).to(device)
        for _ in range(2):  # twice: buffers are reused between calls
            out = spmm.run(xl).cpu().numpy()
            e = sddmm.run(xl, yl).cpu().numpy()
        want = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)[lo:hi]
        np.testing.assert_array_equal(out, want)
        # one exchange shared by both ops
        g = GatheredFeatures(bounds, d, device=device).gather(xl)
        np.testing.assert_array_equal(spmm.run(g).cpu().numpy(), want)
        np.testing.assert_array_equal(sddmm.run(g, yl).cpu().numpy(), e)
        # the same exchange started early and waited for before use
        g2 = GatheredFeatures(bounds, d, device=device)
        g2.gather_async(xl)
        np.testing.assert_array_equal(spmm.run(g2.wait()).cpu().numpy(), want)
        # the exchange as copies into the peers' buffers (symmetric memory), twice: the second exchange must
        # wait for the first one's readers on every rank before it overwrites
        g4 = GatheredFeatures(bounds, d, device=device, peer_copy=True)
        assert g4.exchange == "peer-copy", "symmetric memory could not be set up on this node"
        for _ in range(2):
            g4.gather_async(xl)
            np.testing.assert_array_equal(spmm.run(g4.wait()).cpu().numpy(), want)
            np.testing.assert_array_equal(sddmm.run(g4, yl).cpu().numpy(), e)
        want_e = oracle.sddmm(coo.row, coo.col, x, y)[adj.indptr[lo]:adj.indptr[hi]]
        np.testing.assert_allclose(e, want_e, rtol=1e-5, atol=1e-4)
        # host-buffer step: rows come from pinned host memory, results go back to it (twice: buffers reused)
        from featgraph_b200 import sharded
        xh, yh = torch.from_numpy(x[lo:hi].copy()).pin_memory(), torch.from_numpy(y[lo:hi].copy()).pin_memory()
        oh = torch.empty((hi - lo, d)).pin_memory()
        eh = torch.empty((len(want_e),)).pin_memory()
        g3 = GatheredFeatures(bounds, d, device=device)
        for _ in range(2):
            oh.zero_()
            eh.zero_()
            g3.gather_from_host_async(xh)
            spmm.run_host(g3, oh)
            sddmm.run_host(g3, yh, eh)
            sharded.host_sync(device)
            np.testing.assert_array_equal(oh.numpy(), want)
            np.testing.assert_array_equal(eh.numpy(), e)
    assert spmm.padded == (graph == "power-law"), (graph, bounds)
    if graph == "r-mat":
        # the exchange of only the rows each shard references, over NCCL (all-to-all of the requested rows)
        from featgraph_b200.sharded import NeededFeatures, NeededRows, needed_rows_pay
        rows = NeededRows(local, bounds, device=device)
        assert rows.n_compact < n and needed_rows_pay(rows) in (True, False)
        spmm2 = ShardedSpMM(local, bounds, device=device, needed_rows=rows)
        sddmm2 = ShardedSDDMM(local, bounds, device=device, needed_rows=rows)
        d = 64
        x = graphgen.uniform_features((n, d), seed=81)
        y = graphgen.uniform_features((n, d), seed=82)
        xl = torch.from_numpy(x[lo:hi].copy()).to(device)
        yl = torch.from_numpy(y[lo:hi].copy()).to(device)
        spmm2.build(d)
        sddmm2.build(d)
        gx, gy = NeededFeatures(rows, d, device=device), NeededFeatures(rows, d, device=device)
        for _ in range(2):
            gx.gather_async(xl)
            gy.gather_async(yl)
            h = spmm2.run(gx.wait())
            e2 = sddmm2.run(gy.wait(), h)  # scores against the aggregate, as in the R-MAT step
        want_h = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
        np.testing.assert_array_equal(h.cpu().numpy(), want_h[lo:hi])
        want_e2 = oracle.sddmm(coo.row, coo.col, y, want_h)[adj.indptr[lo]:adj.indptr[hi]]
        scale = max(float(np.abs(want_e2).max()), 1.0)
        np.testing.assert_allclose(e2.cpu().numpy(), want_e2, rtol=1e-5, atol=1e-4 * scale)
        np.testing.assert_array_equal(spmm2.run(xl).cpu().numpy(), want_h[lo:hi])  # the blocking form
        # the same rows fetched by this rank's own kernel from its peers' memory (symmetric memory, NVLink loads)
        px, py = NeededFeatures(rows, d, device=device, peer_pull=True), NeededFeatures(rows, d, device=device, peer_pull=True)
        assert px.exchange == "peer-pull", "symmetric memory could not be set up on this node"
        for _ in range(2):
            px.gather_async(xl)
            py.gather_async(yl)
            h = spmm2.run(px.wait())
            e3 = sddmm2.run(py.wait(), h)
        np.testing.assert_array_equal(px.full.cpu().numpy(), gx.full.cpu().numpy())
        np.testing.assert_array_equal(h.cpu().numpy(), want_h[lo:hi])
        np.testing.assert_array_equal(e3.cpu().numpy(), e2.cpu().numpy())


def check_full_size_shard(rank, world, device):
    """The benchmarked configuration on this rank's shard: the 232,965-node / 114,615,892-edge power-law
    graph, features exchanged by GatheredFeatures.gather_async / wait (as the benchmark's step does), at
    the narrowest and the widest benchmarked feature length.  Sampled rows of this rank's range (its
    longest included) against the CPU oracle: SpMM bit for bit, SDDMM within rtol 1e-5 / atol 1e-4."""
    import oracle
    from featgraph_b200 import graphgen
    from featgraph_b200.sharded import GatheredFeatures, ShardedSDDMM, ShardedSpMM
    from featgraph_b200.util import nnz_balanced_row_ranges

    w = graphgen.WORKLOADS["C2"]
    n, nnz, seed = w["n"], w["nnz"], w["seed"]
    deg = graphgen.power_law_degrees(n, nnz, seed)
    indptr_all = np.zeros(n + 1, dtype=np.int64)
    np.cumsum(deg, out=indptr_all[1:])
    bounds = nnz_balanced_row_ranges(indptr_all, world)
    lo, hi = int(bounds[rank]), int(bounds[rank + 1])
    local = graphgen.power_law_graph(n, nnz, seed, rows=(lo, hi))
    assert local.nnz == int(indptr_all[hi] - indptr_all[lo])
    spmm = ShardedSpMM(local, bounds, device=device)
    sddmm = ShardedSDDMM(local, bounds, device=device)
    ldeg = np.diff(local.indptr)
    rng = np.random.default_rng(500 + rank)
    rows = np.unique(np.concatenate([rng.integers(0, hi - lo, 200), np.argsort(-ldeg)[:4], [0, hi - lo - 1]]))
    sub_ptr = np.zeros(len(rows) + 1, dtype=np.int32)
    np.cumsum(ldeg[rows], out=sub_ptr[1:])
    idx = np.concatenate([np.arange(local.indptr[r], local.indptr[r + 1]) for r in rows])
    sub_cols = local.indices[idx]
    row_of = np.repeat(rows + lo, ldeg[rows]).astype(np.int32)  # global row ids
    for d in (32, 512):
        x = graphgen.workload_features("C2", n, d, 0)
        y = graphgen.workload_features("C2", n, d, 1)
        xl = torch.from_numpy(np.ascontiguousarray(x[lo:hi])).to(device)
        yl = torch.from_numpy(np.ascontiguousarray(y[lo:hi])).to(device)
        spmm.build(d)
        sddmm.build(d)
        g = GatheredFeatures(bounds, d, device=device)
        for _ in range(2):  # twice: the exchange buffer and the outputs are reused between steps
            g.gather_async(xl)
            g.wait()
            out = spmm.run(g).cpu().numpy()
            e = sddmm.run(g, yl).cpu().numpy()
        want = oracle.spmm_csr(sub_ptr, sub_cols, local.data[idx], x)
        np.testing.assert_array_equal(out[rows], want)
        want_e = oracle.sddmm(row_of, sub_cols, x, y)  # column side x (gathered), row side y (local rows)
        np.testing.assert_allclose(e[idx], want_e, rtol=1e-5, atol=1e-4)
        del g


if __name__ == "__main__":
    main()
