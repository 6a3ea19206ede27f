"""DRAM traffic per library call, from one ncu pass, for the benchmark's roofline.

Step 1, on a B200, under ncu (profiling starts and stops around the measured calls only):

    ncu --profile-from-start off --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum \\
        --clock-control none --csv --log-file traffic.csv \\
        python -m featgraph_b200.benchmark.ncu_traffic --run --counts counts.json

  runs SpMM and SDDMM once (after one warm-up call each) at every feature length on the 232,965-node /
  114,615,892-edge power-law graph and writes, per call, how many kernels the library launched.

Step 2, anywhere:

    python -m featgraph_b200.benchmark.ncu_traffic --summarise traffic.csv --counts counts.json \\
        --out profiles/ncu_traffic.json

  splits ncu's launch list by those counts and writes DRAM bytes per call together with the kernels'
  compile-time signature (fg_kernel_signature), which bench.py compares with the loaded library's before it
  trusts the table.
"""
import argparse
import csv
import json

DIMS = (32, 64, 128, 256, 512)


def run(counts_path, dims):
    import torch
    from featgraph import placeholder
    from featgraph.module import VanillaSDDMMcuda, VanillaSpMMcuda
    from featgraph_b200 import _native, graphgen
    L = _native.lib()
    adj = graphgen.workload_graph("C2")
    n = adj.shape[0]
    spmm, sddmm = VanillaSpMMcuda(adj), VanillaSDDMMcuda(adj.tocoo())
    calls = []
    for d in dims:
        x = torch.from_numpy(graphgen.workload_features("C2", n, d, 0)).cuda()
        y = torch.from_numpy(graphgen.workload_features("C2", n, d, 1)).cuda()
        spmm.build([placeholder((n, d))], {}, {})
        sddmm.build([placeholder((n, d)), placeholder((n, d))], {}, {})
        for op, fn in (("spmm", lambda: spmm.run([x])), ("sddmm", lambda: sddmm.run([x, y]))):
            fn()  # warm-up, not profiled
            torch.cuda.synchronize()
            before = L.fg_kernel_launch_count()
            torch.cuda.profiler.start()
            fn()
            torch.cuda.synchronize()
            torch.cuda.profiler.stop()
            calls.append({"op": op, "d": d, "launches": int(L.fg_kernel_launch_count() - before)})
    json.dump({"kernel_signature": L.fg_kernel_signature().decode(), "calls": calls}, open(counts_path, "w"))
    print("ok: %d calls, %d launches" % (len(calls), sum(c["launches"] for c in calls)))


def summarise(csv_path, counts_path, out_path):
    counts = json.load(open(counts_path))
    rows = [r for r in csv.reader(open(csv_path)) if len(r) > 8]
    hdr = rows[0]
    k_id, k_name, k_metric, k_val = (hdr.index(c) for c in ("ID", "Kernel Name", "Metric Name", "Metric Value"))
    launches = {}  # ncu launch id -> {"name": ..., metric: value}
    for r in rows[1:]:
        e = launches.setdefault(int(r[k_id]), {"name": r[k_name]})
        e[r[k_metric]] = float(r[k_val].replace(",", ""))
    ordered = [launches[i] for i in sorted(launches)]
    units = {}
    for r in rows[1:]:
        units[r[k_metric]] = r[hdr.index("Metric Unit")]
    scale = {"byte": 1.0, "Kbyte": 1e3, "Mbyte": 1e6, "Gbyte": 1e9, "Tbyte": 1e12}
    at, out = 0, []
    for c in counts["calls"]:
        part = ordered[at:at + c["launches"]]
        at += c["launches"]
        assert len(part) == c["launches"], "ncu saw fewer launches than the library counted"
        dram = sum(p["dram__bytes_read.sum"] * scale[units["dram__bytes_read.sum"]] +
                   p["dram__bytes_write.sum"] * scale[units["dram__bytes_write.sum"]] for p in part)
        out.append({"op": c["op"], "d": c["d"], "launches": c["launches"], "dram_bytes_per_call": dram,
                    "kernels": sorted({p["name"].split("(")[0].replace("void <unnamed>::", "") for p in part})})
    assert at == len(ordered), "ncu saw %d launches, the library counted %d" % (len(ordered), at)
    json.dump({"kernel_signature": counts["kernel_signature"], "captured_by":
               "ncu --profile-from-start off --metrics dram__bytes_read.sum,dram__bytes_write.sum,gpu__time_duration.sum "
               "--clock-control none; python -m featgraph_b200.benchmark.ncu_traffic --run",
               "workload": "C2/C3 power-law graph 232965 nodes / 114615892 edges, one call per (op, d)",
               "calls": out}, open(out_path, "w"), indent=1)
    for e in out:
        print("%-5s d=%3d launches=%d dram=%.2f GB" % (e["op"], e["d"], e["launches"], e["dram_bytes_per_call"] / 1e9))


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--run", action="store_true")
    ap.add_argument("--summarise", default=None, metavar="NCU_CSV")
    ap.add_argument("--counts", required=True)
    ap.add_argument("--out", default="profiles/ncu_traffic.json")
    ap.add_argument("--dims", default=",".join(str(d) for d in DIMS))
    a = ap.parse_args()
    if a.run:
        run(a.counts, [int(v) for v in a.dims.split(",")])
    if a.summarise:
        summarise(a.summarise, a.counts, a.out)
