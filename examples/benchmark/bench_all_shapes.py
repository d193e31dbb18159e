#!/usr/bin/env python
"""Sweep the fused GEMM + collective examples over a shape list and 1 / 2 / 4 / 8 ranks.

Role in the reference: ``examples/benchmark/bench_all_shapes.py:11-277`` (one SLURM job per shape and GPU count,
tile sizes looked up in ``dataset/tiling.json``).  Here every point is a local multi-process run started with
``iris_b200.launch``; each writes one JSON file, and points whose file already exists are skipped, so an
interrupted sweep resumes where it stopped.

    python examples/benchmark/bench_all_shapes.py --input_json configs/shapes.json --out results/sweep --gpus 1 2 4 8
"""
import argparse
import json
import os
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
SCRIPTS = {"all_scatter": "examples/07_gemm_all_scatter/benchmark.py",
           "atomic": "examples/08_gemm_atomics_all_reduce/benchmark.py",
           "one_shot": "examples/09_gemm_one_shot_all_reduce/benchmark.py",
           "two_shot": "examples/09_gemm_one_shot_all_reduce/benchmark.py"}


def tiling_for(table, m, n, k):
    cfg = dict(table["default"])
    for o in table.get("overrides", []):
        if (o["m"], o["n"], o["k"]) == (m, n, k):
            cfg.update({k_: v for k_, v in o.items() if k_ not in ("m", "n", "k")})
    return cfg


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--input_json", default=os.path.join(ROOT, "configs", "shapes.json"))
    ap.add_argument("--tiling_json", default=os.path.join(ROOT, "configs", "tiling_b200.json"))
    ap.add_argument("--out", default=os.path.join(ROOT, "results", "sweep"))
    ap.add_argument("--gpus", type=int, nargs="+", default=[1, 2, 4, 8])
    ap.add_argument("--only", nargs="*", default=None, help="restrict to these shape names")
    ap.add_argument("--timeout", type=float, default=300.0, help="seconds per point (the reference uses 5 minutes)")
    ap.add_argument("--dry_run", "-n", action="store_true")
    args = ap.parse_args()
    with open(args.input_json) as f:
        shapes = json.load(f)["shapes"]
    with open(args.tiling_json) as f:
        table = json.load(f)
    os.makedirs(args.out, exist_ok=True)
    for s in shapes:
        if args.only and s["name"] not in args.only:
            continue
        for workload in s["workloads"]:
            for w in args.gpus:
                m, n, k = s["m"], s["n"], s["k"]
                if workload == "all_scatter" and n % w:
                    continue
                if workload != "all_scatter" and (k % w or (k // w) % 8):
                    continue
                per_rank = (m, n // w, k) if workload == "all_scatter" else (m, n, k // w)
                cfg = tiling_for(table, *per_rank)
                out = os.path.join(args.out, f"{s['name']}_{workload}_w{w}.json")
                if os.path.exists(out):
                    print(f"skip {out} (exists)")
                    continue
                cmd = [sys.executable, "-m", "iris_b200.launch", "-np", str(w), "--timeout", str(args.timeout),
                       os.path.join(ROOT, SCRIPTS[workload]), "-m", str(m), "-n", str(n), "-k", str(k), "-v", "-b",
                       "--gsize_m", str(cfg["gsize_m"]), "--gemm_sms", str(cfg["gemm_sms"]), "--output_file", out]
                if workload in ("atomic", "one_shot", "two_shot") and workload != "atomic":
                    cmd += ["--variant", workload]
                print(" ".join(cmd), flush=True)
                if not args.dry_run:
                    subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT))


if __name__ == "__main__":
    main()
