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
    p.add_argument("--exchange", choices=("auto", "collective", "peer"), default="auto",
                   help="N > 1: how the feature rows are exchanged. collective: the backend's all-gather / all-to-all. "
                        "peer: through symmetric memory - one device-to-device copy per peer (all-gather layouts; copy "
                        "engines, no SMs), or each rank reading the rows it needs from its peers' memory (needed-rows "
                        "layout). auto: peer for the needed-rows layout (C4) and, up to 4 GPUs, for the all-gather layouts; "
                        "collective otherwise")
    p.add_argument("--all-gather", action="store_true",
                   help="C4 at N > 1: exchange whole feature matrices (all-gather) even where exchanging only the rows "
                        "each shard references would be chosen")
    p.add_argument("--fused", action="store_true",
                   help="C4 on one GPU: the fused aggregate-then-score call instead of SpMM followed by SDDMM")
    p.add_argument("--e2e-steps", type=int, default=4)
    p.add_argument("--e2e-tiled-sddmm", action="store_true",
                   help="end-to-end leg on one GPU: SDDMM through column windows of feature tiles even where the "
                        "one-pass kernel over column blocks would be used")
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
SDDMM_SAMPLE_DIV = 64  # the single-threaded SDDMM is timed on the first nnz / 64 edges
SPMM_SAMPLE_DIV = 4    # the all-threads SpMM on the first n / 4 rows (rows are independent, degrees i.i.d.)


class CpuStep:
    """One bounded sample of the step on the host cores, as the reference's x86 path would run it: at
    EVERY feature length of the step, SpMM on the first quarter of the rows with every host thread
    (row-parallel, with the layout copies the reference's timed function contains,
    python/featgraph/op/vanilla_spmm.py:41-62) and SDDMM on ONE thread (the reference's x86 SDDMM schedule
    has no parallel loop, python/featgraph/op/vanilla_sddmm.py:66-74) on the first nnz / 64 edges.  The
    step rate is formed from all feature lengths: FLOPs of a full step / (sum of the SpMM and SDDMM sample
    times, each scaled to the whole graph)."""

    def __init__(self, adj, dims):
        import oracle
        from featgraph_b200 import graphgen
        self.oracle, self.adj, self.dims = oracle, adj, dims
        n = adj.shape[0]
        self.ne = max(1, adj.nnz // SDDMM_SAMPLE_DIV)
        self.row = np.repeat(np.arange(n, dtype=np.int32), np.diff(adj.indptr))[:self.ne]
        self.col = adj.indices[:self.ne]
        self.x = {d: graphgen.workload_features(WORKLOAD, n, d, 0) for d in dims}
        self.y = {d: graphgen.workload_features(WORKLOAD, n, d, 1) for d in dims}
        self.rows = max(1, n // SPMM_SAMPLE_DIV)
        self.sub_ptr = np.ascontiguousarray(adj.indptr[:self.rows + 1])
        self.sub_nnz = int(self.sub_ptr[-1])
        self.out = {d: np.empty((self.rows, d), dtype=np.float32) for d in dims}
        self.oe = np.empty(self.ne, dtype=np.float32)
        self.threads = oracle.num_threads()

    def run(self):
        """One pass over every feature length; returns {d: (spmm seconds, sddmm sample seconds)}."""
        o, adj, t = self.oracle, self.adj, {}
        for d in self.dims:
            t0 = time.perf_counter()
            o.spmm_csr(self.sub_ptr, adj.indices[:self.sub_nnz], adj.data[:self.sub_nnz], self.x[d], with_copies=True,
                       out=self.out[d])
            t1 = time.perf_counter()
            o.sddmm(self.row, self.col, self.x[d], self.y[d], threads=1, out=self.oe)
            t[d] = (t1 - t0, time.perf_counter() - t1)
        return t

    def summarise(self, runs):
        """Mean times over ``runs`` (a list of run() results) -> rates."""
        nnz, scale = self.adj.nnz, self.adj.nnz / float(self.ne)
        scale_spmm = nnz / float(max(self.sub_nnz, 1))
        per_d, est_step, sample = {}, 0.0, 0.0
        for d in self.dims:
            ts = float(np.mean([r[d][0] for r in runs]))
            te = float(np.mean([r[d][1] for r in runs]))
            per_d[d] = {"spmm_sample_s": ts, "spmm_gflops": 2.0 * self.sub_nnz * d / ts / 1e9,
                        "sddmm_sample_s": te, "sddmm_gflops": 2.0 * self.ne * d / te / 1e9}
            est_step += ts * scale_spmm + te * scale
            sample += ts + te
        flops = sum(2 * 2.0 * nnz * d for d in self.dims)
        return {"step_gflops": flops / est_step / 1e9, "estimated_full_step_s": est_step, "sample_s": sample,
                "per_d": per_d, "threads": self.threads, "sddmm_edges": self.ne, "spmm_rows": self.rows,
                "spmm_nnz": self.sub_nnz}

    def extras(self, d=64):
        """Variants that are not the reference's schedule, once each at one feature length: SpMM with
        dynamic row scheduling and no layout copies, SDDMM with OpenMP over edges, and scipy's csr.dot on one
        thread (the ground truth of the reference's own tests, tests/test_module_spmm.py:29)."""
        o, adj = self.oracle, self.adj
        d = d if d in self.dims else self.dims[0]

        def timed(fn):
            t0 = time.perf_counter()
            fn()
            return time.perf_counter() - t0

        t_dyn = timed(lambda: o.spmm_csr(self.sub_ptr, adj.indices[:self.sub_nnz], adj.data[:self.sub_nnz], self.x[d],
                                         dynamic=True, out=self.out[d]))
        t_mt = timed(lambda: o.sddmm(self.row, self.col, self.x[d], self.y[d], threads=self.threads, out=self.oe))
        rows = max(1, adj.shape[0] // 8)  # scipy is single-threaded: an eighth of the rows bounds its time
        sub = adj[:rows]
        t_sp = timed(lambda: sub.dot(self.x[d]))
        return {"d": d, "spmm_dynamic_nocopy_gflops": 2.0 * self.sub_nnz * d / t_dyn / 1e9,
                "sddmm_openmp_gflops": 2.0 * self.ne * d / t_mt / 1e9,
                "scipy_csr_dot_1thread_gflops": 2.0 * sub.nnz * d / t_sp / 1e9, "scipy_rows": rows}

    def sample_text(self):
        return ("at each d in %s: SpMM on the first %d rows (%d nonzeros; all %d threads, with the reference's layout "
                "copies); SDDMM on one thread (the reference's x86 SDDMM has no parallel loop) on the first %d edges; "
                "both scaled to the whole graph; rate = FLOPs of a full step / estimated full-step time"
                % (self.dims, self.rows, self.sub_nnz, self.threads, self.ne))


def workload_text(n, nnz):
    return ("C4 R-MAT graph %d nodes / %d edges: H = A.X then out[e] = dot(H[row e], Y[col e])"
            if WORKLOAD == "C4" else
            "C2/C3 power-law graph %d nodes / %d edges: SpMM + SDDMM at each d") % (n, nnz)


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
    dims = [int(x) for x in args.dims.split(",")]
    step = CpuStep(adj, dims)
    # each "step" is one bounded sample of the whole step (every feature length)
    for _ in range(max(args.warmup, 0)):
        step.run()
    t0 = time.perf_counter()
    runs = [step.run() for _ in range(max(args.steps, 1))]
    wall = time.perf_counter() - t0
    r = step.summarise(runs)
    r["extras"] = step.extras()
    line = {
        "impl": "reference", "metric": "spmm_sddmm_gflops", "value": r["step_gflops"], "unit": "GFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": 1e3 * wall / max(args.steps, 1),
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_text(n, nnz), "dims": dims,
                   "note": "host cores only (no GPU is used, whatever --gpus says): the CPU restatement of the "
                           "reference's x86 path (the reference itself needs a code generator that is not "
                           "installed). ms_per_step is the wall time of one bounded sample; value is the rate of "
                           "the full step formed from it: " + step.sample_text()},
        "cpu_baseline": {"value": r["step_gflops"], "unit": "GFLOP/s", "cores": r["threads"], "kind": "port",
                         "sample": step.sample_text(), "detail": r},
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

    # C4 at N > 1: a shard of the R-MAT graph references a fraction of the feature rows, so only those are
    # exchanged (all-to-all of the requested rows) where that pays; C2's rows reference nearly every column.
    needed = None
    if WORKLOAD == "C4" and world > 1 and not args.all_gather:
        from featgraph_b200.sharded import NeededRows, needed_rows_pay
        cand = NeededRows(local_adj, bounds, device=device)
        log("[rank %d] needs %d of %d feature rows (%.2f)" % (rank, cand.n_compact, n, cand.fraction()))
        if needed_rows_pay(cand):
            needed = cand
    spmm = ShardedSpMM(local_adj, bounds, device=device, needed_rows=needed)
    sddmm = ShardedSDDMM(local_adj, bounds, device=device, needed_rows=needed)

    def exchange_buffer(d):
        if needed is not None:
            from featgraph_b200.sharded import NeededFeatures
            return NeededFeatures(needed, d, device=device, peer_pull=args.exchange in ("auto", "peer"))
        return GatheredFeatures(bounds, d, device=device)

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
    # copy-engine exchange where it was measured to pay (2 and 4 GPUs); at ~360 GB/s per GPU the largest exchange
    # of a step would no longer hide behind the kernels of a 1/8 shard, so from 8 GPUs on the collective is used
    peer_copy = args.exchange == "peer" or (args.exchange == "auto" and 1 < world <= 4)
    shared = {d: GatheredFeatures(bounds, d, device=device, peer_copy=peer_copy) for d in dims} \
        if WORKLOAD != "C4" else {}
    # C4 at N > 1: Y is not needed before the SDDMM, so its exchange runs beside the SpMM
    c4_y = {d: exchange_buffer(d) for d in dims} if WORKLOAD == "C4" and world > 1 else {}
    c4_x = {d: exchange_buffer(d) for d in dims} if WORKLOAD == "C4" and world > 1 else {}
    exchange_kind = shared[dims[0]].exchange if shared else \
        ("needed-rows / " + c4_x[dims[0]].exchange if (needed is not None and c4_x) else "all-gather")
    c4_pull = bool(c4_x) and getattr(c4_x[dims[0]], "exchange", "") == "peer-pull"
    if c4_pull:
        # the step's inputs live where the peers can read them (this rank's block of the symmetric buffers):
        # resident before the timed region like every other input, and the exchange copies nothing locally
        for d in dims:
            for buf, t in ((c4_x[d], dev_feats[d][0]), (c4_y[d], dev_feats[d][1])):
                buf.local_input.copy_(t)
            dev_feats[d] = (c4_x[d].local_input, c4_y[d].local_input)
        torch.cuda.synchronize(device)

    prefetch = world > 1 and WORKLOAD != "C4" and not args.no_prefetch
    c4_overlap = bool(c4_y) and not args.no_prefetch

    fused = None
    if args.fused:
        if WORKLOAD != "C4" or world != 1:
            raise SystemExit("--fused is the one-GPU C4 step")
        from featgraph import placeholder as _ph
        from featgraph_b200.module import AggregateThenScore
        fused = AggregateThenScore(local_adj, device=device)
        fused.build([_ph((n, dims[0])), _ph((n, dims[0]))])

    def step(record=None):
        if fused is not None:  # one call does both ops: its time is booked under "spmm", "sddmm" stays 0
            for d in dims:
                xd, yd = dev_feats[d]
                ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if record is not None else None
                if ev:
                    ev[0].record(stream)
                    ev[1].record(stream)
                fused.run([xd, yd])
                if ev:
                    for k in (2, 3, 4):
                        ev[k].record(stream)
                    record.append((d, ev))
            return
        if prefetch:  # every feature matrix of the step is resident: exchange d[k+1] while d[k] computes
            shared[dims[0]].gather_async(dev_feats[dims[0]][0])
        for k, d in enumerate(dims):
            xd, yd = dev_feats[d]
            spmm.build_cached(d, args.feat_tile)
            sddmm.build_cached(d)
            ev = [torch.cuda.Event(enable_timing=True) for _ in range(5)] if record is not None else None
            if ev:
                ev[0].record(stream)
            if WORKLOAD == "C4" and world > 1:
                # X's exchange, then (beside the SpMM, unless --no-prefetch) Y's
                c4_x[d].gather_async(xd)
                if c4_overlap and not c4_pull:
                    c4_y[d].gather_async(yd)
                gx = c4_x[d].wait()
                if c4_overlap and c4_pull:
                    c4_y[d].gather_async(yd)  # its reads start when X's have ended: beside the SpMM, not beside X
                if ev:
                    ev[1].record(stream)
                h = spmm.run(gx)
                if ev:
                    ev[2].record(stream)
                if not c4_overlap:
                    c4_y[d].gather_async(yd)
                gy = c4_y[d].wait()
                if ev:
                    ev[3].record(stream)
                sddmm.run(gy, h)  # column side Y (exchanged), row side H = A.X (local rows)
            elif WORKLOAD == "C4":
                spmm.gather(xd)
                if ev:
                    ev[1].record(stream)
                h = spmm.compute()
                if ev:
                    ev[2].record(stream)
                sddmm.gather(yd)
                if ev:
                    ev[3].record(stream)
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

    # --- order-independent checksum of every output's bits, summed over ranks ---------------------
    # (taken from the device-timed steps' outputs, before the end-to-end leg reuses the buffers)
    # SpMM sums every element in storage order and SDDMM's tree is fixed per edge, so these values must
    # be the same at every GPU count (the sharded outputs concatenate to the single-GPU output).
    checksums = {}
    for d in dims:
        outs = (("spmm", fused.out), ("sddmm", fused.scores)) if fused is not None else \
            (("spmm", spmm.out_cache[d][0]), ("sddmm", sddmm.out_cache[d][0]))
        for op, t in outs:
            c = t.contiguous().view(torch.int32).to(torch.int64).sum().reshape(1)
            if world > 1:
                dist.all_reduce(c, op=dist.ReduceOp.SUM)
            checksums["%s_d%d" % (op, d)] = int(c.item())

    # --- end to end: host buffers in, host result out, every step -------------------------------
    e2e = None
    if not args.no_e2e and fused is None:
        from featgraph_b200 import sharded
        outs_host = {d: (torch.empty((hi - lo, d), dtype=torch.float32).pin_memory(),
                         torch.empty((local_nnz,), dtype=torch.float32).pin_memory()) for d in dims}
        # bytes copied per step, counted from the tensors the step copies
        if WORKLOAD == "C4":
            h2d = sum(2 * (hi - lo) * d * 4 for d in dims) + (sum((hi - lo) * d * 4 for d in dims) if world == 1 else 0)
        else:
            h2d = sum(2 * (hi - lo) * d * 4 for d in dims)  # X_d once (shared by both ops) and Y_d
        d2h = sum((hi - lo) * d * 4 + local_nnz * 4 for d in dims)

        def e2e_step():
            if world == 1:
                for d in dims:
                    xh, yh = feats[d]
                    # the library's host-buffer calls: copies pipelined against the kernels
                    if WORKLOAD == "C4":  # the second op consumes the first one's host result
                        spmm.build_cached(d, args.feat_tile)
                        sddmm.build_cached(d)
                        hh = spmm.module.run_host([xh], out=outs_host[d][0])
                        sddmm.module.run_host([yh, hh], out=outs_host[d][1])
                    else:  # deferred completion: one call's copy-out overlaps the next call
                        # (the SDDMM scores the features the SpMM call has just uploaded: X goes over PCIe once)
                        e2e_mod[("spmm", d)].run_host([xh], out=outs_host[d][0], wait=False)
                        e2e_mod[("sddmm", d)].run_host([e2e_mod[("spmm", d)].device_input, yh], out=outs_host[d][1],
                                                       wait=False)
                featgraph_b200.host_sync(device)
                stream.synchronize()
                return
            # N > 1: the sharded layer's host-buffer calls.  Every copy-in and the exchange behind it are
            # issued first (they need only the copy-in stream), then the kernels, each followed by its
            # copy-out on the copy-out stream: a step costs about max(copies in, kernels, copies out).
            for d in dims:
                if WORKLOAD == "C4":  # copy this rank's rows in, then start both exchanges behind the copies
                    s_in, _ = sharded.copy_streams(device)
                    xs, ys = c4_stage[d]
                    with torch.cuda.stream(s_in):
                        for buf in (e2e_x[d], e2e_y[d]):  # peer-pull: the stage is the block the peers read from
                            if getattr(buf, "local_input", None) is not None:
                                buf.wait_writable()
                        xs.copy_(feats[d][0], non_blocking=True)
                        ys.copy_(feats[d][1], non_blocking=True)
                        e2e_x[d].gather_async(xs)
                        e2e_y[d].gather_async(ys)
                else:
                    e2e_x[d].gather_from_host_async(feats[d][0])
            for d in dims:
                spmm.build_cached(d, args.feat_tile)
                sddmm.build_cached(d)
                if WORKLOAD == "C4":
                    sharded.wait_for_copy_out(spmm.module.out, device, spmm)
                    h = spmm.run(e2e_x[d].wait())
                    sharded.copy_out_async(h, outs_host[d][0], device, spmm)
                    sharded.wait_for_copy_out(sddmm.module.out, device, sddmm)
                    o2 = sddmm.run(e2e_y[d].wait(), h)
                    sharded.copy_out_async(o2, outs_host[d][1], device, sddmm)
                else:
                    spmm.run_host(e2e_x[d], outs_host[d][0])
                    sddmm.run_host(e2e_x[d], feats[d][1], outs_host[d][1])
            sharded.host_sync(device)

        e2e_mod, e2e_x, e2e_y, c4_stage = {}, {}, {}, {}
        if world > 1:
            e2e_x = {d: exchange_buffer(d) for d in dims}
            if WORKLOAD == "C4":
                e2e_y = {d: exchange_buffer(d) for d in dims}
                def stage(buf, d):
                    own = getattr(buf, "local_input", None)
                    return own if own is not None else torch.empty((hi - lo, d), device=device)
                c4_stage = {d: (stage(e2e_x[d], d), stage(e2e_y[d], d)) for d in dims}
        elif WORKLOAD != "C4":
            # deferred calls must not share staging buffers: one module per (op, d) for the e2e leg
            from featgraph import placeholder as _ph
            from featgraph.module import VanillaSDDMMcuda as _SD, VanillaSpMMcuda as _SP
            coo_local = local_adj.tocoo()
            for d in dims:
                m1 = _SP(local_adj, device=device)
                m1.build([_ph((n, d))], {}, {})
                m2 = _SD(coo_local, device=device)
                m2.build([_ph((n, d)), _ph((n, d))], {}, {"col_blocks": 1} if args.e2e_tiled_sddmm else {})
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
                       "copied from pinned host memory and results read back every step; "
                       + ("through run_host (fg_*_host: column windows pipelined, completion deferred to the end of the step)"
                          if world == 1 else
                          "through the sharded layer's host-buffer calls (gather_from_host_async / run_host: "
                          "copy-in and exchange of every feature matrix issued ahead of the kernels, results "
                          "leaving on a copy-out stream)")}

    # --- per-kernel table and roofline (per GPU: whole-graph bytes / N over the slowest rank's time) --
    peak, peak_kind = measured_peak_gbs()
    traffic_table, traffic_note = load_ncu_traffic(_native.lib().fg_kernel_signature().decode())
    kernels = []
    for (op, d), ts in sorted(per_kernel.items()):
        ms = float(np.mean(ts))
        g_ms = float(np.mean(gather_ms[(op, d)]))
        if world > 1:
            t = torch.tensor([ms, g_ms], device=device, dtype=torch.float64)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms, g_ms = float(t[0].item()), float(t[1].item())
        bt = bytes_touched(n, nnz, d) / world  # this GPU's share (rows and nonzeros are split evenly)
        touched = bt / (ms * 1e-3) / 1e9
        dram = traffic_table.get((op, d))
        kernels.append({
            "op": op, "d": d, "ms": ms, "all_gather_ms": g_ms if world > 1 else 0.0,
            "gflops": 2.0 * nnz * d / (ms * 1e-3) / 1e9,
            "touched_gbs_per_gpu": touched, "frac_touched": touched / peak,
            "l2_frac": touched / L2_TO_SM_PEAK_GBS,
            "dram_bytes": dram, "dram_frac": (dram / (ms * 1e-3) / 1e9 / peak) if (dram and world == 1) else None,
            "frac_compulsory": bytes_unique(n, n, nnz, d) / world / (ms * 1e-3) / 1e9 / peak,
            "checksum": checksums["%s_d%d" % (op, d)],
        })
    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return
    dom = max(kernels, key=lambda k: k["ms"])
    roofline = {
        "bound": "hbm", "kernel": "%s d=%d (one library call)" % (dom["op"], dom["d"]),
        "achieved": dom["touched_gbs_per_gpu"], "peak": peak, "unit": "GB/s", "frac": dom["frac_touched"],
        "peak_kind": "of " + peak_kind,
        "traffic": dom["dram_bytes"] if world == 1 else None,
        "dram_frac": dom["dram_frac"], "l2_frac": dom["l2_frac"], "l2_peak_gbs": L2_TO_SM_PEAK_GBS,
        "compulsory_frac": dom["frac_compulsory"],
        "algorithmic_bytes": bytes_touched(n, nnz, dom["d"]) / world,
        "traffic_source": traffic_note,
        "note": "per GPU. achieved = touched bytes (every nonzero fetches index, value and its feature-row slice) "
                "/ kernel time: the gathered part of the feature matrix is sized to stay in L2, so this exceeds "
                "the HBM peak by design; dram_frac = DRAM bytes per call seen by ncu / time / HBM peak is what "
                "HBM delivers, l2_frac = touched bytes / time / the L2-to-SM rate the ncu captures imply "
                "(20.6 TB/s at lts__throughput 88 %) is how close the kernel is to the path that bounds it",
    }
    if world > 1:
        roofline["note"] += "; N > 1: whole-graph bytes / N over the slowest rank's kernel time"
    line = {
        "metric": "spmm_sddmm_gflops", "value": value, "unit": "GFLOP/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": workload_text(n, nnz),
                   "dims": dims, "parallelism": "row-sharded x%d (nnz-balanced); each feature matrix all-gathered "
                   "once per step and d, inside the timed region%s" % (world, ", the exchange for the next d running beside "
                   "the current d's kernels" if prefetch else
                                                  (", Y's exchange running beside the SpMM" if c4_overlap else "")) +
                   ("; only the rows each shard references are exchanged" if needed is not None else "")
                   if world > 1 else "single GPU",
                   "l2_policy": "inputs larger than L2 (CSR arrays %.0f MB per pass; 10 different kernels "
                                "and feature matrices between repeats of any one)" % (8.0 * nnz / 1e6),
                   "exchange": exchange_kind if world > 1 else None,
                   "feat_tile": args.feat_tile or "auto", "fused_call": bool(fused is not None),
                   "kernel_signature": _native.lib().fg_kernel_signature().decode()},
        "roofline": roofline, "kernels": kernels, "checksums": checksums, "e2e": e2e,
        "gpu_launches": launches, "clocks": clocks,
    }
    if not args.no_cpu_baseline and world == 1:
        t0 = time.time()
        cpu = CpuStep(local_adj, dims)
        cpu.run()  # warm-up
        r = cpu.summarise([cpu.run()])
        r["extras"] = cpu.extras()
        line["cpu_baseline"] = {
            "value": r["step_gflops"], "unit": "GFLOP/s", "cores": r["threads"], "kind": "port",
            "sample": cpu.sample_text() + "; 1 warm-up + 1 timed pass", "detail": r, "wall_s": time.time() - t0}
    emit(line)
    if world > 1:
        dist.destroy_process_group()


# The L2 -> SM delivery rate the ncu captures of the SpMM rows kernel imply: 20.6 TB/s delivered at
# lts__throughput 88 % of peak (profiles/spmm_rows_kernel_c2.md).
L2_TO_SM_PEAK_GBS = 20600.0 / 0.88


def load_ncu_traffic(signature):
    """DRAM bytes per library call (dram__bytes_read.sum + dram__bytes_write.sum summed over the call's
    launches) from profiles/ncu_traffic.json, keyed by (op, d) - but only if that file was captured from
    kernels of the same compile-time shapes as the ones loaded now (fg_kernel_signature)."""
    path = os.path.join(ROOT, "profiles", "ncu_traffic.json")
    try:
        rec = json.load(open(path))
    except Exception:
        return {}, "profiles/ncu_traffic.json absent"
    if rec.get("kernel_signature") != signature:
        return {}, "profiles/ncu_traffic.json is stale: captured from kernels %r, loaded %r" % (
            rec.get("kernel_signature"), signature)
    table = {(e["op"], int(e["d"])): float(e["dram_bytes_per_call"]) for e in rec.get("calls", [])}
    return table, "profiles/ncu_traffic.json (%s)" % rec.get("captured_by", "ncu")


def _install_build_cache(spmm, sddmm):
    """Keep one built state (output, gather buffer, plan) per feature length so that switching d inside
    a step neither allocates nor re-plans."""
    cache_a, cache_b = {}, {}
    spmm_keys = ("out", "_feat_shape", "_feat_tile")
    sddmm_keys = ("out", "_shapes", "_feat_tile", "_exact", "_plan")

    def build_spmm(d, tile=0):
        if d not in cache_a:
            spmm.build(d, tile)
            cache_a[d] = tuple(getattr(spmm.module, k) for k in spmm_keys) + (spmm.x_full,)
        for k, v in zip(spmm_keys, cache_a[d]):
            setattr(spmm.module, k, v)
        spmm.x_full = cache_a[d][-1]

    def build_sddmm(d):
        if d not in cache_b:
            sddmm.build(d)
            cache_b[d] = tuple(getattr(sddmm.module, k) for k in sddmm_keys) + (sddmm.src_full,)
        for k, v in zip(sddmm_keys, cache_b[d]):
            setattr(sddmm.module, k, v)
        sddmm.src_full = cache_b[d][-1]

    spmm.build_cached, spmm.out_cache = build_spmm, cache_a
    sddmm.build_cached, sddmm.out_cache = build_sddmm, cache_b


if __name__ == "__main__":
    a = parse_args()
    if a.dims is None:
        a.dims = "128" if a.workload == "C4" else "32,64,128,256,512"
    WORKLOAD = a.workload
    if a.impl == "reference":
        run_reference_arm(a)
    else:
        run_ours(a)
