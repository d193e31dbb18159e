#!/usr/bin/env python
"""GEMM + one-shot all-reduce (K-sharded): partial tiles stay local, per-tile flags, every rank pulls and sums all partials; --variant two_shot lets one owner per tile sum and push (examples/09_gemm_one_shot_all_reduce/benchmark.py of the reference).

    python -m iris_b200.launch -np 8 examples/09_gemm_one_shot_all_reduce/benchmark.py -v -b
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.gemm_driver import run  # noqa: E402

if __name__ == "__main__":
    run("one_shot", seed=3)
