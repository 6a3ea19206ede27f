"""The module layer on the GPU, written the way the reference's own tests are
(tests/test_module_spmm.py, tests/test_module_sddmm.py): same matrix shape, feature length,
knob tuples and scipy / numpy ground truth, plus the oracle."""
import numpy as np
import pytest
import scipy.sparse as sp
import torch

from conftest import ATOL, RTOL
from featgraph import placeholder
from featgraph.module import VanillaSDDMMcuda, VanillaSDDMMx86, VanillaSpMMcuda, VanillaSpMMx86

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def adj_csr():
    return sp.random(127, 255, density=0.1, format="csr", random_state=42).astype("float32")


@pytest.fixture(scope="module")
def adj_coo():
    return sp.random(127, 255, density=0.1, format="coo", random_state=43).astype("int32")


@pytest.mark.parametrize("feat_len,num_col_partitions,num_feat_partitions", [(128, 1, 1), (128, 4, 1), (128, 4, 4)])
def test_vanilla_spmm_x86(oracle, adj_csr, feat_len, num_col_partitions, num_feat_partitions):
    num_rows, num_cols = adj_csr.shape
    module = VanillaSpMMx86(adj_csr, num_col_partitions)
    SrcFeat = placeholder((num_cols, feat_len))
    module.build([SrcFeat], {'num_feat_partitions': num_feat_partitions}, {})
    src_feat_np = np.random.default_rng(0).random((num_cols, feat_len), dtype=np.float32)
    out = module.run([torch.from_numpy(src_feat_np).to(module.ctx)]).cpu().numpy()
    np.testing.assert_allclose(adj_csr.dot(src_feat_np), out, rtol=1e-4, atol=1e-4)
    if num_col_partitions == 1:
        want = oracle.spmm_csr(adj_csr.indptr, adj_csr.indices, adj_csr.data, src_feat_np,
                               num_feat_partitions=num_feat_partitions)
    else:
        from featgraph.util import util_convert_csr_to_dds
        want = oracle.spmm_dds(*util_convert_csr_to_dds(adj_csr, num_col_partitions), src_feat_np, num_rows,
                               num_col_partitions, num_feat_partitions=num_feat_partitions)
    np.testing.assert_array_equal(out, want)
    assert module.target == 'llvm'


@pytest.mark.parametrize("num_threads_per_cuda_block", [32, 128, None])
def test_vanilla_spmm_cuda(oracle, adj_csr, num_threads_per_cuda_block):
    num_rows, num_cols = adj_csr.shape
    module = VanillaSpMMcuda(adj_csr)
    SrcFeat = placeholder((num_cols, 128))
    module.build([SrcFeat], {}, {'num_threads_per_cuda_block': num_threads_per_cuda_block})
    src_feat_np = np.random.default_rng(1).random((num_cols, 128), dtype=np.float32)
    out_t = module.run([torch.from_numpy(src_feat_np).to(module.ctx)])
    out = out_t.cpu().numpy()
    np.testing.assert_allclose(adj_csr.dot(src_feat_np), out, rtol=1e-4, atol=1e-4)
    np.testing.assert_array_equal(out, oracle.spmm_csr(adj_csr.indptr, adj_csr.indices, adj_csr.data, src_feat_np))
    # destination passing: the same tensor comes back on every run
    assert module.run([torch.from_numpy(src_feat_np).to(module.ctx)]) is out_t
    assert module.target == 'cuda' and module.ctx.type == 'cuda'
    assert module.measure_average_time([torch.from_numpy(src_feat_np).to(module.ctx)], 3) > 0
    assert "fg_spmm_csr_f32" in module.lower_to_ir([SrcFeat], {}, {})


def test_spmm_accepts_coo_input_and_run_host(adj_csr):
    module = VanillaSpMMcuda(adj_csr.tocoo())
    module.build([placeholder((255, 64))], {}, {})
    x = np.random.default_rng(2).random((255, 64), dtype=np.float32)
    out = module.run_host([x])
    np.testing.assert_allclose(adj_csr.dot(x), out.numpy(), rtol=1e-4, atol=1e-4)


@pytest.mark.parametrize("d,chunk", [(64, 0), (256, 0), (256, 32), (200, 64), (136, 0)])
def test_host_buffer_calls_pipeline_windows_and_match_device_calls(oracle, d, chunk):
    """run_host (copies pipelined over column windows) against run on device tensors, with pinned and
    with pageable host memory."""
    from featgraph_b200 import graphgen
    adj = graphgen.power_law_graph(4000, 300_000, seed=51, kmax=3000)
    n = adj.shape[0]
    x = graphgen.uniform_features((n, d), seed=52)
    y = graphgen.uniform_features((n, d), seed=53)
    sp_ = VanillaSpMMcuda(adj)
    sp_.build([placeholder((n, d))], {}, {})
    want = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
    got_pageable = sp_.run_host([x], chunk=chunk).numpy().copy()
    np.testing.assert_array_equal(got_pageable, want)
    pinned_out = torch.empty((n, d)).pin_memory()
    got = sp_.run_host([torch.from_numpy(x).pin_memory()], out=pinned_out, chunk=chunk)
    assert got is pinned_out
    np.testing.assert_array_equal(got.numpy(), want)
    coo = adj.tocoo()
    sd = VanillaSDDMMcuda(coo)
    sd.build([placeholder((n, d)), placeholder((n, d))], {}, {})
    e = sd.run_host([x, y], chunk=chunk).numpy()
    np.testing.assert_allclose(e, oracle.sddmm(coo.row, coo.col, x, y), rtol=RTOL, atol=ATOL)
    with pytest.raises(ValueError):
        sp_.run_host([x[:, :8].copy()])
    # deferred completion: both calls are only enqueued; results are complete after host_sync()
    import featgraph_b200
    o1 = torch.zeros((n, d)).pin_memory()
    o2 = torch.zeros((coo.nnz,)).pin_memory()
    xp, yp = torch.from_numpy(x).pin_memory(), torch.from_numpy(y).pin_memory()
    sp_.run_host([xp], out=o1, chunk=chunk, wait=False)
    sd.run_host([xp, yp], out=o2, chunk=chunk, wait=False)
    # a module with a deferred call in flight refuses further calls (its staging buffers are in use)
    with pytest.raises(RuntimeError, match="deferred"):
        sp_.run_host([xp], out=o1, chunk=chunk, wait=False)
    with pytest.raises(RuntimeError, match="deferred"):
        sd.run([torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()])
    featgraph_b200.host_sync()
    np.testing.assert_array_equal(o1.numpy(), want)
    np.testing.assert_allclose(o2.numpy(), oracle.sddmm(coo.row, coo.col, x, y), rtol=RTOL, atol=ATOL)
    # the SDDMM host call takes the features the SpMM host call has just uploaded, without copying them again
    sp_.run_host([xp], out=o1, chunk=chunk, wait=False)
    o3 = torch.zeros((coo.nnz,)).pin_memory()
    sd.run_host([sp_.device_input, yp], out=o3, chunk=chunk, wait=False)
    featgraph_b200.host_sync()
    np.testing.assert_array_equal(o3.numpy(), o2.numpy())
    # with column blocks planned, the resident form runs the one-pass kernel (same dot products to rounding)
    sd.build([placeholder((n, d)), placeholder((n, d))], {}, {"col_blocks": 3})
    if sd._plan is not None:
        sp_.run_host([xp], out=o1, chunk=chunk, wait=False)
        sd.run_host([sp_.device_input, yp], out=o3, wait=False)
        featgraph_b200.host_sync()
        np.testing.assert_allclose(o3.numpy(), oracle.sddmm(coo.row, coo.col, x, y), rtol=RTOL, atol=ATOL)
    sd.build([placeholder((n, d)), placeholder((n, d))], {}, {})
    # ... and is usable again after host_sync()
    np.testing.assert_array_equal(sp_.run_host([xp], out=o1, chunk=chunk).numpy(), want)


def test_spmm_build_and_run_argument_errors(adj_csr):
    module = VanillaSpMMcuda(adj_csr)
    with pytest.raises(TypeError):
        module.build([placeholder((255, 64))], {'num_feat_partitions': 2}, {})  # not a cuda compute arg
    with pytest.raises(ValueError):
        module.build([placeholder((254, 64))], {}, {})
    with pytest.raises(RuntimeError):
        module.run([torch.zeros(255, 64, device=module.ctx)])
    module.build([placeholder((255, 64))], {}, {})
    with pytest.raises(ValueError):
        module.run([torch.zeros(255, 32, device=module.ctx)])
    with pytest.raises(TypeError):
        module.run([torch.zeros(255, 64, device=module.ctx, dtype=torch.float64)])
    with pytest.raises(ValueError):
        VanillaSpMMx86(adj_csr, 2).build([placeholder((255, 30))], {'num_feat_partitions': 4}, {})
    with pytest.raises(AssertionError):
        VanillaSpMMx86(adj_csr, 0)


@pytest.mark.parametrize("feat_len,num_feat_partitions,num_row_partitions,num_col_partitions",
                         [(128, 1, 1, 1), (128, 4, 1, 1), (128, 4, 4, 4)])
def test_vanilla_sddmm_x86(oracle, adj_coo, feat_len, num_feat_partitions, num_row_partitions, num_col_partitions):
    adj = adj_coo.copy()
    num_rows, num_cols = adj.shape
    module = VanillaSDDMMx86(adj, num_row_partitions, num_col_partitions)
    SrcFeat = placeholder((num_cols, feat_len))
    DstFeat = placeholder((num_rows, feat_len))
    module.build([SrcFeat, DstFeat], {'num_feat_partitions': num_feat_partitions},
                 {'num_feat_partitions': num_feat_partitions})
    rng = np.random.default_rng(3)
    src_feat_np = rng.random((num_cols, feat_len), dtype=np.float32)
    dst_feat_np = rng.random((num_rows, feat_len), dtype=np.float32)
    out = module.run([torch.from_numpy(src_feat_np).to(module.ctx),
                      torch.from_numpy(dst_feat_np).to(module.ctx)]).cpu().numpy()
    if num_row_partitions != 1 or num_col_partitions != 1:
        out = out[module.edge_mapping]
    out_numpy = (src_feat_np[adj.col] * dst_feat_np[adj.row]).sum(axis=-1)
    np.testing.assert_allclose(out_numpy, out, rtol=1e-4, atol=1e-4)
    # the x86 class keeps the x86 loop's summation order: bit-identical to the oracle
    np.testing.assert_array_equal(out, oracle.sddmm(adj.row, adj.col, src_feat_np, dst_feat_np,
                                                    num_feat_partitions=num_feat_partitions))


@pytest.mark.parametrize("num_cuda_blocks", [32, 256])
def test_vanilla_sddmm_cuda(oracle, adj_coo, num_cuda_blocks):
    num_rows, num_cols = adj_coo.shape
    module = VanillaSDDMMcuda(adj_coo)
    SrcFeat = placeholder((num_cols, 128))
    DstFeat = placeholder((num_rows, 128))
    module.build([SrcFeat, DstFeat], {}, {'num_cuda_blocks': num_cuda_blocks})
    rng = np.random.default_rng(4)
    src_feat_np = rng.random((num_cols, 128), dtype=np.float32)
    dst_feat_np = rng.random((num_rows, 128), dtype=np.float32)
    ins = [torch.from_numpy(src_feat_np).to(module.ctx), torch.from_numpy(dst_feat_np).to(module.ctx)]
    out = module.run(ins).cpu().numpy()
    out_numpy = (src_feat_np[adj_coo.col] * dst_feat_np[adj_coo.row]).sum(axis=-1)
    np.testing.assert_allclose(out_numpy, out, rtol=1e-4, atol=1e-4)
    np.testing.assert_allclose(out, oracle.sddmm(adj_coo.row, adj_coo.col, src_feat_np, dst_feat_np),
                               rtol=RTOL, atol=ATOL)
    assert module.measure_average_time(ins, 3) > 0
    with pytest.raises(AssertionError):
        module.edge_mapping  # no partitioning on cuda
    with pytest.raises(AssertionError):
        module.build([SrcFeat, DstFeat], {}, {'num_cuda_blocks': adj_coo.nnz + 1})


def test_sddmm_quirk_column_partitions_follow_row_argument(adj_coo):
    """python/featgraph/module/sddmm.py:37: num_col_partitions is overwritten by num_row_partitions."""
    m = VanillaSDDMMx86(adj_coo.copy(), 1, 4)
    with pytest.raises(AssertionError):
        m.edge_mapping  # 1 x 1 after the overwrite: not partitioned
    m = VanillaSDDMMx86(adj_coo.copy(), 3, 1)
    assert m.edge_mapping.shape == (adj_coo.nnz,) and m.edge_mapping.dtype == np.int64


@pytest.mark.parametrize("world", [1, 3, 8])
def test_row_shards_on_one_gpu_reproduce_the_whole_graph(oracle, world):
    """The per-rank work of the multi-GPU layer, run shard after shard on one GPU: remapped column ids
    gathering from the padded buffer give the rows / edges of the single-GPU result, bit for bit (SpMM)."""
    from featgraph_b200 import graphgen
    from featgraph_b200.sharded import padded_layout, remap_columns_to_padded, shard_csr_rows
    from featgraph_b200.util import nnz_balanced_row_ranges
    n, d = 3000, 64
    adj = graphgen.power_law_graph(n, 200_000, seed=21, kmax=2500)
    x = graphgen.uniform_features((n, d), seed=22)
    y = graphgen.uniform_features((n, d), seed=23)
    bounds = nnz_balanced_row_ranges(adj.indptr, world)
    slot, shift = padded_layout(bounds)
    padded = np.zeros((world * slot, d), dtype=np.float32)
    for p in range(world):
        lo, hi = int(bounds[p]), int(bounds[p + 1])
        padded[p * slot:p * slot + hi - lo] = x[lo:hi]
    padded_dev = torch.from_numpy(padded).cuda()
    want = oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x)
    coo = adj.tocoo()
    want_e = oracle.sddmm(coo.row, coo.col, x, y)
    for p in range(world):
        lo, hi = int(bounds[p]), int(bounds[p + 1])
        local = remap_columns_to_padded(shard_csr_rows(adj, bounds, p), bounds)
        m = VanillaSpMMcuda(local)
        m.build([placeholder((world * slot, d))], {}, {})
        np.testing.assert_array_equal(m.run([padded_dev]).cpu().numpy(), want[lo:hi])
        s = VanillaSDDMMcuda(local.tocoo())
        s.build([placeholder((world * slot, d)), placeholder((hi - lo, d))], {}, {})
        got = s.run([padded_dev, torch.from_numpy(y[lo:hi].copy()).cuda()]).cpu().numpy()
        np.testing.assert_allclose(got, want_e[adj.indptr[lo]:adj.indptr[hi]], rtol=RTOL, atol=ATOL)


def test_sharded_wrappers_single_process(oracle):
    """ShardedSpMM / ShardedSDDMM without a process group (world size 1)."""
    from featgraph_b200 import graphgen
    from featgraph_b200.sharded import ShardedSDDMM, ShardedSpMM
    from featgraph_b200.util import nnz_balanced_row_ranges
    n, d = 1500, 32
    adj = graphgen.power_law_graph(n, 60_000, seed=31, kmax=900)
    x = graphgen.uniform_features((n, d), seed=32)
    y = graphgen.uniform_features((n, d), seed=33)
    bounds = nnz_balanced_row_ranges(adj.indptr, 1)
    sp_ = ShardedSpMM(adj, bounds)
    sp_.build(d)
    out = sp_.run(torch.from_numpy(x).cuda()).cpu().numpy()
    np.testing.assert_array_equal(out, oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x))
    sd = ShardedSDDMM(adj, bounds)
    sd.build(d)
    e = sd.run(torch.from_numpy(x).cuda(), torch.from_numpy(y).cuda()).cpu().numpy()
    coo = adj.tocoo()
    np.testing.assert_allclose(e, oracle.sddmm(coo.row, coo.col, x, y), rtol=RTOL, atol=ATOL)


def test_benchmark_scripts_read_npz_datasets(tmp_path):
    """The reference's benchmarks take --dataset <scipy .npz> (CSR for SpMM, COO for SDDMM, as
    benchmark/download_reddit_dataset.py:13,17 writes them); the counterparts here read the same files."""
    import subprocess
    import sys
    from conftest import ROOT
    adj = sp.random(300, 300, density=0.05, format="csr", random_state=7).astype("float32")
    csr_path, coo_path = str(tmp_path / "g_csr.npz"), str(tmp_path / "g_coo.npz")
    sp.save_npz(csr_path, adj)
    sp.save_npz(coo_path, adj.tocoo())
    for mod, path, target in (("bench_vanilla_spmm", csr_path, "cuda"), ("bench_vanilla_spmm", csr_path, "x86"),
                              ("bench_vanilla_sddmm", coo_path, "cuda")):
        r = subprocess.run([sys.executable, "-m", "featgraph_b200.benchmark." + mod, "--dataset", path,
                            "--feat-len", "32", "--target", target], capture_output=True, text=True, cwd=ROOT,
                           timeout=600)
        assert r.returncode == 0, r.stderr[-2000:]
        assert "average time of 5 runs" in r.stdout
    # one rank's rows of a several-GPU run
    r = subprocess.run([sys.executable, "-m", "featgraph_b200.benchmark.bench_vanilla_spmm", "--dataset", csr_path,
                        "--feat-len", "32", "--shard", "1/3"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    assert "shard 1 of 3" in r.stdout and "average time of 5 runs" in r.stdout


def test_sddmm_module_column_blocks(oracle):
    """``col_blocks``: the one-pass traversal over column blocks gives the dot products of the tiled call,
    in the caller's edge order; an edge list that is not in CSR order quietly takes the tiled call."""
    from featgraph_b200 import graphgen
    adj = graphgen.power_law_graph(400, 400 * 30, seed=17, kmax=350)
    coo = adj.tocoo()
    n, d = 400, 256
    src, dst = graphgen.uniform_features((n, d), seed=18), graphgen.uniform_features((n, d), seed=19)
    want = oracle.sddmm(coo.row, coo.col, src, dst)
    m = VanillaSDDMMcuda(coo)
    s, t = torch.from_numpy(src).to(m.ctx), torch.from_numpy(dst).to(m.ctx)
    m.build([placeholder((n, d)), placeholder((n, d))], {}, {})
    assert m._plan is None  # small enough for L2: nothing to block
    plain = m.run([s, t]).cpu().numpy().copy()
    m.build([placeholder((n, d)), placeholder((n, d))], {}, {"col_blocks": 5})
    assert m._plan is not None
    blocked = m.run([s, t]).cpu().numpy()
    np.testing.assert_allclose(blocked, want, rtol=RTOL, atol=ATOL)
    np.testing.assert_allclose(blocked, plain, rtol=RTOL, atol=ATOL)
    assert m.measure_average_time([s, t], 2) > 0
    # shuffled edge list: no plan can be built, the result is still right and in the caller's order
    perm = np.random.default_rng(1).permutation(coo.nnz)
    import scipy.sparse as sp
    shuffled = sp.coo_matrix((coo.data[perm], (coo.row[perm], coo.col[perm])), shape=coo.shape)
    m2 = VanillaSDDMMcuda(shuffled)
    m2.build([placeholder((n, d)), placeholder((n, d))], {}, {"col_blocks": 5})
    assert m2._plan is None
    np.testing.assert_allclose(m2.run([s, t]).cpu().numpy(), want[perm], rtol=RTOL, atol=ATOL)
