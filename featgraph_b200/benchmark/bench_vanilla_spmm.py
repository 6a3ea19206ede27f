"""Knob sweep for vanilla SpMM on a graph stored as a scipy .npz (CSR), the counterpart of the
reference's benchmark/bench_vanilla_spmm.py: same flags (--dataset --feat-len --target), same
sweeps, same protocol (mean seconds of 5 back-to-back runs after a warm-up).  Both targets run on
the GPU here; 'x86' sweeps the x86 class's partition knobs, 'cuda' the CUDA class's launch knobs
(accepted, no effect on results or, by design, on speed) plus the feature-tile width.

Without --dataset a seeded synthetic graph is generated (--synthetic C0|C1|C2|C4).  --shard R/W keeps
only the rows that rank R of W owns (nnz-balanced contiguous ranges, all columns): what one GPU of a
W-GPU run computes.
"""
import argparse
import os
import sys

import numpy as np
import scipy.sparse
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from featgraph import placeholder  # noqa: E402
from featgraph.module import VanillaSpMMcuda, VanillaSpMMx86  # noqa: E402


def exp_range(start, end, mul):
    while start <= end:
        yield start
        start *= mul


def time_once(module, placeholders, compute_args, schedule_args, num_cols, feat_len, num_runs=5):
    module.build(placeholders, compute_args, schedule_args)
    x = torch.rand((num_cols, feat_len), dtype=torch.float32, device=module.ctx)
    return module.measure_average_time([x], num_runs)


def bench_x86(adj, feat_len):
    num_cols = adj.shape[1]
    for num_col_partitions in exp_range(1, 32, 2):
        module = VanillaSpMMx86(adj, num_col_partitions)
        for num_feat_partitions in exp_range(1, max(feat_len // 16, 1), 2):
            if feat_len % num_feat_partitions:
                continue
            t = time_once(module, [placeholder((num_cols, feat_len))],
                          {'num_feat_partitions': num_feat_partitions}, {}, num_cols, feat_len)
            print("num_col_partitions: %d  num_feat_partitions: %d  average time of 5 runs: %.6f sec"
                  % (num_col_partitions, num_feat_partitions, t))


def bench_cuda(adj, feat_len):
    num_rows, num_cols = adj.shape
    module = VanillaSpMMcuda(adj)
    for feat_tile in (0, 32, 64, 128):
        if feat_tile > max(feat_len, 4):
            continue
        t = time_once(module, [placeholder((num_cols, feat_len))], {}, {'feat_tile': feat_tile}, num_cols, feat_len)
        print("feat_tile: %s  average time of 5 runs: %.4f ms  (%.0f GFLOP/s)"
              % (feat_tile or "auto", t * 1e3, 2.0 * adj.nnz * feat_len / t / 1e9))
    for num_cuda_blocks in exp_range(64, num_rows, 4):
        t = time_once(module, [placeholder((num_cols, feat_len))], {},
                      {'num_cuda_blocks': num_cuda_blocks, 'num_threads_per_cuda_block': min(feat_len, 32)},
                      num_cols, feat_len)
        print("num_cuda_blocks: %d  average time of 5 runs: %.4f ms" % (num_cuda_blocks, t * 1e3))


if __name__ == '__main__':
    parser = argparse.ArgumentParser()
    parser.add_argument("--dataset", type=str, help="The adjacency matrix in csr format stored as a scipy npz file")
    parser.add_argument("--synthetic", type=str, default="C0", help="named synthetic graph when no --dataset is given")
    parser.add_argument("--feat-len", type=int, default=128, help="The feature length")
    parser.add_argument("--target", type=str, default='cuda', choices=['x86', 'cuda'])
    parser.add_argument("--shard", type=str, default=None, help="R/W: only the rows of rank R of W (nnz-balanced ranges)")
    args = parser.parse_args()
    if args.dataset:
        adj = scipy.sparse.load_npz(args.dataset)
        assert adj.format == 'csr'
        adj = scipy.sparse.csr_matrix((adj.data.astype(np.float32), adj.indices.astype(np.int32),
                                       adj.indptr.astype(np.int32)), shape=adj.shape)
    else:
        from featgraph_b200 import graphgen
        adj = graphgen.workload_graph(args.synthetic)
    if args.shard:
        from featgraph_b200.sharded import shard_csr_rows
        from featgraph_b200.util import nnz_balanced_row_ranges
        r, w = (int(v) for v in args.shard.split("/"))
        adj = shard_csr_rows(adj, nnz_balanced_row_ranges(adj.indptr, w), r)
        print("shard %d of %d: %d rows, %d nonzeros" % (r, w, adj.shape[0], adj.nnz))
    (bench_x86 if args.target == 'x86' else bench_cuda)(adj, args.feat_len)
