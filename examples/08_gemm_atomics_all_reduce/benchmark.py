#!/usr/bin/env python
"""GEMM + atomic all-reduce (K-sharded): every partial tile is added into the C of every rank with TMA reduce-adds (examples/08_gemm_atomics_all_reduce/benchmark.py of the reference).

    python -m iris_b200.launch -np 8 examples/08_gemm_atomics_all_reduce/benchmark.py -v -b
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.gemm_driver import run  # noqa: E402

if __name__ == "__main__":
    run("atomic", seed=3)
