"""Knob sweep for vanilla SDDMM on a graph stored as a scipy .npz (COO), the counterpart of the
reference's benchmark/bench_vanilla_sddmm.py (same flags, sweeps and timing protocol).  Both targets
run on the GPU here.  Without --dataset a seeded synthetic graph is generated.
"""
import argparse
import os
import sys

import numpy as np
import scipy.sparse
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from featgraph import placeholder  # noqa: E402
from featgraph.module import VanillaSDDMMcuda, VanillaSDDMMx86  # noqa: E402


def exp_range(start, end, mul):
    while start <= end:
        yield start
        start *= mul


def time_once(module, shapes, compute_args, schedule_args, num_runs=5):
    module.build([placeholder(s) for s in shapes], compute_args, schedule_args)
    ins = [torch.rand(s, dtype=torch.float32, device=module.ctx) for s in shapes]
    return module.measure_average_time(ins, num_runs)


def bench_x86(adj, feat_len):
    num_rows, num_cols = adj.shape
    for num_row_partitions in exp_range(1, 32, 2):
        module = VanillaSDDMMx86(adj.copy(), num_row_partitions, num_row_partitions)
        for num_feat_partitions in exp_range(1, max(feat_len // 16, 1), 2):
            if feat_len % num_feat_partitions:
                continue
            t = time_once(module, [(num_cols, feat_len), (num_rows, feat_len)],
                          {'num_feat_partitions': num_feat_partitions}, {'num_feat_partitions': num_feat_partitions})
            print("num_row_partitions: %d  num_col_partitions: %d  num_feat_partitions: %d  "
                  "average time of 5 runs: %.6f sec" % (num_row_partitions, num_row_partitions, num_feat_partitions, t))


def bench_cuda(adj, feat_len):
    num_rows, num_cols = adj.shape
    module = VanillaSDDMMcuda(adj)
    for feat_tile in (0, 32, 64, 128, 256, 512):
        if feat_tile > max(feat_len, 4):
            continue
        t = time_once(module, [(num_cols, feat_len), (num_rows, feat_len)], {}, {'feat_tile': feat_tile})
        print("feat_tile: %s  average time of 5 runs: %.4f ms  (%.0f GFLOP/s)"
              % (feat_tile or "auto", t * 1e3, 2.0 * adj.nnz * feat_len / t / 1e9))
    for num_cuda_blocks in exp_range(64, min(262144, adj.nnz // 32), 4):
        t = time_once(module, [(num_cols, feat_len), (num_rows, feat_len)], {}, {'num_cuda_blocks': num_cuda_blocks})
        print("num_cuda_blocks: %d  average time of 5 runs: %.4f ms" % (num_cuda_blocks, t * 1e3))


if __name__ == '__main__':
    parser = argparse.ArgumentParser()
    parser.add_argument("--dataset", type=str, help="The adjacency matrix in coo format stored as a scipy npz file")
    parser.add_argument("--synthetic", type=str, default="C1", help="named synthetic graph when no --dataset is given")
    parser.add_argument("--feat-len", type=int, default=128, help="The feature length")
    parser.add_argument("--target", type=str, default='cuda', choices=['x86', 'cuda'])
    args = parser.parse_args()
    if args.dataset:
        adj = scipy.sparse.load_npz(args.dataset)
        assert adj.format == 'coo'
        adj = scipy.sparse.coo_matrix((adj.data.astype(np.int32), (adj.row.astype(np.int32), adj.col.astype(np.int32))),
                                      shape=adj.shape)
    else:
        from featgraph_b200 import graphgen
        adj = graphgen.workload_graph(args.synthetic).tocoo()
    (bench_x86 if args.target == 'x86' else bench_cuda)(adj, args.feat_len)
