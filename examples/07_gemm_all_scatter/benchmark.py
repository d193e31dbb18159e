#!/usr/bin/env python
"""GEMM + all-scatter (tensor-parallel, B column-sharded): every finished C tile is pushed into the C of every rank (examples/07_gemm_all_scatter/benchmark.py of the reference).

    python -m iris_b200.launch -np 8 examples/07_gemm_all_scatter/benchmark.py -v -b
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.gemm_driver import run  # noqa: E402

if __name__ == "__main__":
    run("all_scatter", seed=2)
