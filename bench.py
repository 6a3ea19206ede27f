#!/usr/bin/env python
"""Benchmark of the vanilla SpMM / SDDMM hot path on the 232,965-node / 114,615,892-edge
power-law graph (the stand-in for the Reddit adjacency the reference's benchmarks load).

One STEP = SpMM and SDDMM once at every feature length in --dims (default 32,64,128,256,512) on
that graph: 10 kernel launches.  FLOPs per step = sum_d 2 ops x 2*nnz*d.

    python bench.py [--gpus N] [--steps K] [--warmup W]            # this library on N GPUs
    python bench.py --impl reference [--steps K] [--warmup W]      # the CPU restatement, host cores

N > 1 is launched under torch.distributed.run (one rank per GPU): the graph's rows are split in
nnz-balanced ranges (strong scaling: same graph, more GPUs), feature rows are all-gathered
inside the timed step.  Rank 0 prints ONE JSON line.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = "C2"
N_NODES = 232_965
N_EDGES = 114_615_892


def log(*a):
    print(*a, file=sys.stderr, flush=True)


_JSON_FD = None


def protect_stdout():
    """Keep stdout for the one JSON line: libraries that chat on fd 1 (NCCL prints its version
    banner there) are sent to stderr instead."""
    global _JSON_FD
    if _JSON_FD is None:
        sys.stdout.flush()
        _JSON_FD = os.dup(1)
        os.dup2(2, 1)


def emit(line):
    data = (json.dumps(line) + "\n").encode()
    if _JSON_FD is None:
        sys.stdout.write(data.decode())
        sys.stdout.flush()
    else:
        os.write(_JSON_FD, data)


def parse_args():
    p = argparse.ArgumentParser()
    p.add_argument("--gpus", type=int, default=1)
    p.add_argument("--steps", type=int, default=20)
    p.add_argument("--warmup", type=int, default=3)
    p.add_argument("--impl", default="ours", choices=["ours", "reference"])
    p.add_argument("--dims", default=None, help="feature lengths (default 32,64,128,256,512; 128 for C4)")
    p.add_argument("--workload", default="C2", choices=["C2", "C4"],
                   help="C2: power-law graph, SpMM and SDDMM at each d (the headline); C4: R-MAT scale 22, "
                        "H = A.X then out[e] = dot(H[row e], Y[col e]) at d = 128")
    p.add_argument("--shrink", type=int, default=1, help="divide node count (debug / profiling runs)")
    p.add_argument("--feat-tile", type=int, default=0)
    p.add_argument("--no-e2e", action="store_true")
    p.add_argument("--no-prefetch", action="store_true",
                   help="N > 1: exchange each feature matrix right before its ops instead of during the previous ones")
    p.add_argument("--no-cpu-baseline", action="store_true")
    p.add_argument("--e2e-steps", type=int, default=2)
    return p.parse_args()


def graph_params(shrink):
    if shrink == 1:
        return N_NODES, N_EDGES, 20000
    n = N_NODES // shrink
    return n, N_EDGES // (shrink * shrink), max(20000 // shrink, 8)


def bytes_touched(n_rows, nnz, d):
    """Gather-traffic model: every nonzero fetches its index, value and feature-row slice; every
    row its position and its output (SpMM) / row-side feature row (SDDMM)."""
    return 4 * (n_rows + 1) + 8 * nnz + 4 * nnz * d + 4 * n_rows * d


def bytes_unique(n_rows, n_cols, nnz, d):
    return 4 * (n_rows + 1) + 8 * nnz + 4 * n_cols * d + 4 * n_rows * d


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(path))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi clocks / throttle reasons sampled every 200 ms while the timed region runs."""
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index):
        self.rows = []
        self.proc = None
        self.gpu = gpu_index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.gpu), "--query-gpu=" + self.Q, "--format=csv,noheader,nounits",
                 "-lms", "200"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
                for name, v in zip(names, r[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            except Exception:
                pass
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ----------------------------------------------------------------------------------------------
# CPU leg: the oracle (a restatement of the reference's x86 loop nests) timed on host cores.
# ----------------------------------------------------------------------------------------------
def cpu_reference_rates(adj, d, sddmm_edges, runs):
    """GFLOP/s of the restated x86 path on a bounded sample: SpMM on the whole graph at feature
    length d with every host thread (row-parallel, with the layout copies the reference's timed
    function contains); SDDMM single-threaded, as the reference's x86 schedule is, on the first
    ``sddmm_edges`` edges.  One warm-up run each, then the mean of ``runs``."""
    import oracle
    from featgraph_b200 import graphgen
    n = adj.shape[0]
    x = graphgen.workload_features(WORKLOAD, n, d, 0)
    y = graphgen.workload_features(WORKLOAD, n, d, 1)
    out = np.empty((n, d), dtype=np.float32)

    def timed(fn):
        fn()
        t0 = time.perf_counter()
        for _ in range(runs):
            fn()
        return (time.perf_counter() - t0) / runs

    t_spmm = timed(lambda: oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x, with_copies=True, out=out))
    t_spmm_dyn = timed(lambda: oracle.spmm_csr(adj.indptr, adj.indices, adj.data, x, dynamic=True, out=out))
    ne = min(int(sddmm_edges), adj.nnz)
    row = np.repeat(np.arange(n, dtype=np.int32), np.diff(adj.indptr))[:ne]
    col = adj.indices[:ne]
    oe = np.empty(ne, dtype=np.float32)
    t_sddmm = timed(lambda: oracle.sddmm(row, col, x, y, threads=1, out=oe))
    t_sddmm_mt = timed(lambda: oracle.sddmm(row, col, x, y, threads=oracle.num_threads(), out=oe))
    r_spmm = 2.0 * adj.nnz * d / t_spmm / 1e9
    r_sddmm = 2.0 * ne * d / t_sddmm / 1e9
    return {
        "spmm_gflops": r_spmm, "sddmm_gflops": r_sddmm,
        "spmm_dynamic_nocopy_gflops": 2.0 * adj.nnz * d / t_spmm_dyn / 1e9,
        "sddmm_openmp_gflops": 2.0 * ne * d / t_sddmm_mt / 1e9,
        # a step does the same FLOPs in each op, so the step rate is the harmonic mean
        "step_gflops": 2.0 / (1.0 / r_spmm + 1.0 / r_sddmm),
        "seconds": {"spmm": t_spmm, "sddmm_sample": t_sddmm},
        "threads": oracle.num_threads(), "sddmm_edges": ne, "d": d,
    }


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # torch.distributed.run pins OMP_NUM_THREADS=1 for its workers; this arm is meant to use every
    # host thread it can, so undo that before the OpenMP runtime is loaded.
    os.environ["OMP_NUM_THREADS"] = str(len(os.sched_getaffinity(0)))
    protect_stdout()
    from featgraph_b200 import graphgen
    n, nnz, kmax = graph_params(args.shrink)
    t0 = time.time()
    if WORKLOAD == "C4":
        adj = graphgen.rmat_graph(22 - int(np.log2(args.shrink)), 32, graphgen.WORKLOADS[WORKLOAD]["seed"])
        n, nnz = adj.shape[0], adj.nnz
    else:
        adj = graphgen.power_law_graph(n, nnz, graphgen.WORKLOADS[WORKLOAD]["seed"], kmax=kmax)
    log("graph built in %.1fs" % (time.time() - t0))
    d = 64
    sample_edges = nnz // 16
    # warm-up steps and timed steps: each "step" is one bounded sample run
    for _ in range(max(args.warmup - 1, 0)):
        cpu_reference_rates(adj, d, sample_edges, 1)
    t0 = time.perf_counter()
    r = cpu_reference_rates(adj, d, sample_edges, max(args.steps, 1))
    wall = time.perf_counter() - t0
    line = {
        "impl": "reference", "metric": "spmm_sddmm_gflops", "value": r["step_gflops"], "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * (r["seconds"]["spmm"] + r["seconds"]["sddmm_sample"]),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "C2/C3 power-law graph %d nodes / %d edges: SpMM + SDDMM at each d" % (n, nnz),
                   "dims": [int(x) for x in args.dims.split(",")], "sample_dims": [d],
                   "note": "host cores only (no GPU is used, whatever --gpus says): the CPU restatement of the "
                           "reference's x86 path (the reference itself needs a code generator that is not "
                           "installed); each step is a bounded sample, SpMM at d=%d on all host threads and "
                           "SDDMM at d=%d on one thread as in the reference's schedule" % (d, d)},
        "cpu_baseline": {"value": r["step_gflops"], "unit": "GFLOP/s", "cores": r["threads"], "kind": "port",
                         "sample": "SpMM d=%d whole graph; SDDMM d=%d first %d edges" % (d, d, r["sddmm_edges"]),
                         "detail": r},
        "e2e": {"value": r["step_gflops"], "unit": "GFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "wall_s": wall,
    }
    emit(line)


# ----------------------------------------------------------------------------------------------
# GPU leg
# ----------------------------------------------------------------------------------------------
def run_ours(args):
    import torch
    import torch.distributed as dist
    import featgraph_b200
    from featgraph_b200 import _native, graphgen
    from featgraph_b200.sharded import GatheredFeatures, ShardedSDDMM, ShardedSpMM
    from featgraph_b200.util import nnz_balanced_row_ranges

    protect_stdout()
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus %d needs torch.distributed.run with %d ranks" % (args.gpus, args.gpus))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the GPU arm has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    _native.lib()  # fail here, loudly, if the CUDA library is missing

    dims = [int(x) for x in args.dims.split(",")]
    n, nnz, kmax = graph_params(args.shrink)
    seed = graphgen.WORKLOADS[WORKLOAD]["seed"]

    # --- inputs ---
    t0 = time.time()
    if WORKLOAD == "C4":
        # R-MAT: every rank generates the whole graph (seeded, identical) and keeps its rows
        os.environ["OMP_NUM_THREADS"] = str(max(1, len(os.sched_getaffinity(0)) // world))
        from featgraph_b200.sharded import shard_csr_rows
        whole_adj = graphgen.rmat_graph(22 - int(np.log2(args.shrink)), 32, seed)
        n, nnz = whole_adj.shape[0], whole_adj.nnz
        deg = np.diff(whole_adj.indptr).astype(np.int64)
        bounds = nnz_balanced_row_ranges(whole_adj.indptr, world)
        lo, hi = int(bounds[rank]), int(bounds[rank + 1])
        local_adj = shard_csr_rows(whole_adj, bounds, rank)
        if world > 1:
            del whole_adj
    else:
        # power law: every rank derives the degree sequence, then generates only its own rows
        deg = graphgen.power_law_degrees(n, nnz, seed, kmax=kmax)
        indptr_all = np.zeros(n + 1, dtype=np.int64)
        np.cumsum(deg, out=indptr_all[1:])
        bounds = nnz_balanced_row_ranges(indptr_all, world)
        lo, hi = int(bounds[rank]), int(bounds[rank + 1])
        local_adj = graphgen._csr_from_degrees(deg[lo:hi], n, seed + 1, row_offset=lo)
    local_nnz = local_adj.nnz
    log("[rank %d] rows [%d,%d) nnz %d built in %.1fs" % (rank, lo, hi, local_nnz, time.time() - t0))

    spmm = ShardedSpMM(local_adj, bounds, device=device)
    sddmm = ShardedSDDMM(local_adj, bounds, device=device)

    # features: generated whole (seeded), each rank keeps its rows; pinned host copies for e2e
    feats = {}
    for d in dims:
        x = graphgen.workload_features(WORKLOAD, n, d, 0)[lo:hi]
        y = graphgen.workload_features(WORKLOAD, n, d, 1)[lo:hi]
        feats[d] = (torch.from_numpy(np.ascontiguousarray(x)).pin_memory(),
                    torch.from_numpy(np.ascontiguousarray(y)).pin_memory())
    dev_feats = {d: (feats[d][0].to(device), feats[d][1].to(device)) for d in dims}

    stream = torch.cuda.current_stream(device)
    per_kernel = {("spmm", d): [] for d in dims}
    per_kernel.update({("sddmm", d): [] for d in dims})

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    # C2/C3: both ops of a step gather from the same feature matrix X_d, so it is exchanged once per
    # d and shared (GatheredFeatures); C4: X feeds SpMM, Y feeds SDDMM - two exchanges.
    shared = {d: GatheredFeatures(bounds, d, device=device) for d in dims} if WORKLOAD != "C4" else {}
    # C4 at N > 1: Y is not needed before the SDDMM, so its exchange runs beside the SpMM
    c4_y = {d: GatheredFeatures(bounds, d, device=device) for d in dims} if WORKLOAD == "C4" and world > 1 else {}

    prefetch = world > 1 and WORKLOAD != "C4" and not args.no_prefetch
    c4_overlap = bool(c4_y) and not args.no_prefetch

    def step(record=None):
        if prefetch:  # every feature matrix of the step is resident: exchange d[k+1] while d[k] computes
            shared[dims[0]].gather_async(dev_feats[dims[0]][0])
        for k, d in enumerate(dims):
            xd, yd = dev_feats[d]
            spmm.build_cached(d, args.feat_tile)
            sddmm.build_cached(d)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if record is not None else None
            if ev:
                ev[0].record(stream)
            if WORKLOAD == "C4":
                spmm.gather(xd)
                if ev:
                    ev[1].record(stream)
                if c4_overlap:
                    c4_y[d].gather_async(yd)
                h = spmm.compute()
                if ev:
                    ev[2].record(stream)
                # column side Y (gathered), row side H = A.X (local rows)
                if c4_overlap:
                    gy = c4_y[d].wait()
                else:
                    sddmm.gather(yd)
                if ev:
                    ev[3].record(stream)
                if c4_overlap:
                    sddmm.run(gy, h)
                else:
                    sddmm.compute(h)
            else:
                if prefetch:
                    if k + 1 < len(dims):
                        shared[dims[k + 1]].gather_async(dev_feats[dims[k + 1]][0])
                    g = shared[d].wait()
                else:
                    g = shared[d].gather(xd)
                if ev:
                    ev[1].record(stream)
                spmm.run(g)
                if ev:
                    ev[2].record(stream)
                    ev[3].record(stream)
                sddmm.run(g, yd)
            if ev:
                ev[4].record(stream)
                record.append((d, ev))

    # build() allocates; keep one built state per feature length so that a step only launches
    _install_build_cache(spmm, sddmm)

    for _ in range(args.warmup):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    records = []
    launches_before = _native.lib().fg_kernel_launch_count()
    t_start = torch.cuda.Event(enable_timing=True)
    t_stop = torch.cuda.Event(enable_timing=True)
    barrier()
    t_start.record(stream)
    for _ in range(args.steps):
        step(records)
    t_stop.record(stream)
    launches = int(_native.lib().fg_kernel_launch_count() - launches_before)
    barrier()
    clocks = sampler.stop() if rank == 0 else None
    total_ms = t_start.elapsed_time(t_stop)
    gather_ms = {("spmm", d): [] for d in dims}
    gather_ms.update({("sddmm", d): [] for d in dims})
    for d, ev in records:
        gather_ms[("spmm", d)].append(ev[0].elapsed_time(ev[1]))
        per_kernel[("spmm", d)].append(ev[1].elapsed_time(ev[2]))
        gather_ms[("sddmm", d)].append(ev[2].elapsed_time(ev[3]))
        per_kernel[("sddmm", d)].append(ev[3].elapsed_time(ev[4]))
    if world > 1:
        t = torch.tensor([total_ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms = float(t.item())
    ms_per_step = total_ms / args.steps
    flops_per_step = sum(2 * 2.0 * nnz * d for d in dims)
    value = flops_per_step / (ms_per_step * 1e-3) / 1e9

    # --- end to end: host buffers in, host result out, every step -------------------------------
    e2e = None
    if not args.no_e2e:
        outs_host = {d: (torch.empty((hi - lo, d), dtype=torch.float32).pin_memory(),
                         torch.empty((local_nnz,), dtype=torch.float32).pin_memory()) for d in dims}
        h2d = sum(3 * (hi - lo) * d * 4 for d in dims)
        d2h = sum((hi - lo) * d * 4 + local_nnz * 4 for d in dims)

        def e2e_step():
            for d in dims:
                xh, yh = feats[d]
                spmm.build_cached(d, args.feat_tile)
                sddmm.build_cached(d)
                if world == 1:
                    # the library's host-buffer calls: copies pipelined against the kernels
                    if WORKLOAD == "C4":  # the second op consumes the first one's host result
                        hh = spmm.module.run_host([xh], out=outs_host[d][0])
                        sddmm.module.run_host([yh, hh], out=outs_host[d][1])
                    else:  # deferred completion: one call's copy-out overlaps the next call
                        e2e_mod[("spmm", d)].run_host([xh], out=outs_host[d][0], wait=False)
                        e2e_mod[("sddmm", d)].run_host([xh, yh], out=outs_host[d][1], wait=False)
                    continue
                # N > 1: the same three stages with torch streams around the sharded calls (the
                # exchange sits between copy-in and kernel): copies in on s_in, results out on s_out
                xe, se, ye = stage_in[d]
                with torch.cuda.stream(s_in):
                    xe.copy_(xh, non_blocking=True)
                    ev_x = s_in.record_event()
                    se.copy_(xh, non_blocking=True)
                    ye.copy_(yh, non_blocking=True)
                    ev_sy = s_in.record_event()
                stream.wait_event(ev_x)
                o1 = spmm.run(xe)
                ev_k1 = stream.record_event()
                stream.wait_event(ev_sy)
                o2 = sddmm.run(ye, o1) if WORKLOAD == "C4" else sddmm.run(se, ye)
                ev_k2 = stream.record_event()
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_k1)
                    outs_host[d][0].copy_(o1, non_blocking=True)
                    s_out.wait_event(ev_k2)
                    outs_host[d][1].copy_(o2, non_blocking=True)
            if world == 1:
                featgraph_b200.host_sync(device)
            else:
                s_out.synchronize()
            stream.synchronize()

        if world > 1:
            s_in, s_out = torch.cuda.Stream(device), torch.cuda.Stream(device)
            stage_in = {d: tuple(torch.empty((hi - lo, d), dtype=torch.float32, device=device) for _ in range(3))
                        for d in dims}

        # deferred calls must not share staging buffers: one module per (op, d) for the e2e leg
        e2e_mod = {}
        if world == 1 and WORKLOAD != "C4":
            from featgraph import placeholder as _ph
            from featgraph.module import VanillaSDDMMcuda as _SD, VanillaSpMMcuda as _SP
            coo_local = local_adj.tocoo()
            for d in dims:
                m1 = _SP(local_adj, device=device)
                m1.build([_ph((n, d))], {}, {})
                m2 = _SD(coo_local, device=device)
                m2.build([_ph((n, d)), _ph((n, d))], {}, {})
                e2e_mod[("spmm", d)], e2e_mod[("sddmm", d)] = m1, m2

        e2e_step()
        barrier()
        t0 = time.perf_counter()
        for _ in range(args.e2e_steps):
            e2e_step()
        barrier()
        dt = torch.tensor([(time.perf_counter() - t0) / args.e2e_steps], device=device, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(dt, op=dist.ReduceOp.MAX)
            tb = torch.tensor([h2d, d2h], device=device, dtype=torch.float64)
            dist.all_reduce(tb, op=dist.ReduceOp.SUM)
            h2d, d2h = int(tb[0].item()), int(tb[1].item())
        e2e = {"value": flops_per_step / float(dt.item()) / 1e9, "unit": "GFLOP/s",
               "h2d_bytes_per_step": int(h2d), "d2h_bytes_per_step": int(d2h),
               "ms_per_step": 1e3 * float(dt.item()), "steps": args.e2e_steps,
               "note": "adjacency resident (uploaded at construction, as in the reference); features "
                       "copied from pinned host memory and results read back every step"
                       + ("; through run_host (fg_*_host: column windows pipelined, completion deferred to the end of the step)" if world == 1 else "")}

    # --- per-kernel table and roofline (rank-local time, own rows; max over ranks) --------------
    peak, peak_kind = measured_peak_gbs()
    kernels = []
    for (op, d), ts in sorted(per_kernel.items()):
        ms = float(np.mean(ts))
        if world > 1:
            t = torch.tensor([ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        bt = bytes_touched(n, nnz, d)
        g_ms = float(np.mean(gather_ms[(op, d)]))
        if world > 1:
            t = torch.tensor([g_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            g_ms = float(t.item())
        kernels.append({
            "op": op, "d": d, "ms": ms, "all_gather_ms": g_ms if world > 1 else 0.0,
            "gflops": 2.0 * nnz * d / (ms * 1e-3) / 1e9,
            "touched_gbs": bt / (ms * 1e-3) / 1e9, "frac_touched": bt / (ms * 1e-3) / 1e9 / peak,
            "frac_compulsory": bytes_unique(n, n, nnz, d) / (ms * 1e-3) / 1e9 / peak,
        })
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    dom = max(kernels, key=lambda k: k["ms"])
    roofline = {
        "bound": "hbm", "kernel": "%s d=%d (one library call; SDDMM at d>=256 is one launch per 64-float tile)"
        % (dom["op"], dom["d"]),
        "achieved": dom["touched_gbs"], "peak": peak, "unit": "GB/s", "frac": dom["frac_touched"],
        "peak_kind": "of " + peak_kind, "traffic": NCU_TRAFFIC_BYTES.get((dom["op"], dom["d"])),
        "compulsory_frac": dom["frac_compulsory"],
        "algorithmic_bytes": bytes_touched(n, nnz, dom["d"]),
        "note": "achieved = touched bytes (every nonzero fetches index, value and its feature-row slice) / "
                "kernel time; gathers served from L2 make it exceed DRAM traffic, see traffic",
    }
    if world > 1:
        roofline["note"] += "; per-kernel times are the slowest rank's kernel on its shard, with whole-graph bytes"
    line = {
        "metric": "spmm_sddmm_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": ("C4 R-MAT graph %d nodes / %d edges: H = A.X then out[e] = dot(H[row e], Y[col e])"
                                if WORKLOAD == "C4" else
                                "C2/C3 power-law graph %d nodes / %d edges: SpMM + SDDMM at each d") % (n, nnz),
                   "dims": dims, "parallelism": "row-sharded x%d (nnz-balanced); each feature matrix all-gathered "
                   "once per step and d, inside the timed region%s" % (world, ", the exchange for the next d running beside "
                   "the current d's kernels" if prefetch else
                                                  (", Y's exchange running beside the SpMM" if c4_overlap else ""))
                   if world > 1 else "single GPU",
                   "l2_policy": "inputs larger than L2 (CSR arrays %.0f MB per pass; 10 different kernels "
                                "and feature matrices between repeats of any one)" % (8.0 * nnz / 1e6),
                   "feat_tile": args.feat_tile or "auto"},
        "roofline": roofline, "kernels": kernels, "e2e": e2e,
        "gpu_launches": launches, "clocks": clocks,
    }
    if not args.no_cpu_baseline and world == 1:
        t0 = time.time()
        r = cpu_reference_rates(local_adj, 64, nnz // 16, 1)
        line["cpu_baseline"] = {
            "value": r["step_gflops"], "unit": "GFLOP/s", "cores": r["threads"], "kind": "port",
            "sample": "SpMM d=64 whole graph (all threads, with the reference's layout copies); SDDMM d=64 "
                      "first %d edges on one thread (the reference's x86 SDDMM has no parallel loop); "
                      "1 warm-up + 1 timed run each" % r["sddmm_edges"],
            "detail": r, "wall_s": time.time() - t0}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) from the ncu captures
# summarised under profiles/; keyed by (op, feature length).  Absent = not captured.
NCU_TRAFFIC_BYTES = {
    ("spmm", 512): 10.6e9,    # spmm_rows_kernel<16,4,0,1,0>, one launch (8 tiles inside)
    ("spmm", 128): 3.22e9,
    ("sddmm", 512): 25.7e9,   # sddmm_tile_kernel<8,2,4,1,0>: 8 tile launches of 3.21 GB each
    ("sddmm", 128): 7.58e9,   # two tile launches
}


def _install_build_cache(spmm, sddmm):
    """Keep one output / gather buffer per feature length so that switching d inside a step does
    not allocate."""
    cache_a, cache_b = {}, {}

    def build_spmm(d, tile=0):
        if d not in cache_a:
            spmm.build(d, tile)
            cache_a[d] = (spmm.module.out, spmm.x_full, spmm.module._feat_shape, spmm.module._feat_tile)
        spmm.module.out, spmm.x_full, spmm.module._feat_shape, spmm.module._feat_tile = cache_a[d]

    def build_sddmm(d):
        if d not in cache_b:
            sddmm.build(d)
            cache_b[d] = (sddmm.module.out, sddmm.src_full, sddmm.module._shapes)
        sddmm.module.out, sddmm.src_full, sddmm.module._shapes = cache_b[d]

    spmm.build_cached = build_spmm
    sddmm.build_cached = build_sddmm


if __name__ == "__main__":
    a = parse_args()
    if a.dims is None:
        a.dims = "128" if a.workload == "C4" else "32,64,128,256,512"
    WORKLOAD = a.workload
    if a.impl == "reference":
        run_reference_arm(a)
    else:
        run_ours(a)
