#!/usr/bin/env python
"""GEMM + reduce-scatter (K-sharded): every rank keeps its own M / ranks rows of the sum.  Partial tiles are pushed once,
to the rank that keeps their rows, in an order that gives every keeper one sender at a time; the keeper sums from local
memory.  This is the row-parallel projection of a sequence-parallel transformer layer.  The reference has the collective
only as an RCCL baseline (examples/benchmark/reference/reduce_scatter.py); the fused form is an addition.

    python -m iris_b200.launch -np 8 examples/11_gemm_reduce_scatter/benchmark.py -v -b
"""
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.gemm_driver import run  # noqa: E402

if __name__ == "__main__":
    run("reduce_scatter", seed=5)
