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
sys.path.insert(0, ROOT)
from iris_b200.utils.config import GemmPoint, load_points  # noqa: E402


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
    for pt in load_points({"shapes": shapes}, args.gpus):
        if args.only and pt.name not in args.only:
            continue
        why = pt.problems()
        if why:
            print(f"skip {pt.name} {pt.workload} W={pt.world}: {'; '.join(why)}")
            continue
        out = os.path.join(args.out, f"{pt.name}_{pt.workload}_w{pt.world}.json")
        if os.path.exists(out):
            print(f"skip {out} (exists)")
            continue
        cmd = pt.command(ROOT, table, output_file=out, python=sys.executable, timeout_s=args.timeout)
        print(" ".join(cmd), flush=True)
        if not args.dry_run:
            subprocess.run(cmd, cwd=ROOT, env=dict(os.environ, PYTHONPATH=ROOT))

if __name__ == "__main__":
    main()
