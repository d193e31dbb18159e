#!/usr/bin/env python
"""Single-GPU library GEMM throughput (cuBLAS through torch), the denominator the fused kernels are compared
with at one rank (``examples/benchmark/reference/gemm.py:1-31`` of the reference).  Also times this repository's
tcgen05 kernel on the same operands."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _common as C  # noqa: E402
from _common import torch  # noqa: E402


def main():
    args = C.parse_args("library GEMM vs tcgen05 GEMM, one GPU")
    m, n, k = args["m"], args["n"], args["k"]
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(0)
    A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    out = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
    total, _, _ = C.time_two_phase(lambda: torch.matmul(A, Bt.t(), out=out), lambda: None, 1, args["num_warmup"],
                                   args["num_experiments"])
    print(f"cuBLAS   {m}x{n}x{k}: {total * 1e3:.1f} us = {2.0 * m * n * k / total / 1e9:.1f} TFLOPS")
    import iris_b200 as iris
    from iris_b200.ops import gemm as G
    ctx = iris.Iris.local_world(1, heap_size=1 << 20)[0]
    op = G.FusedGemm(ctx, [A], [Bt], "store", out=[out])
    total2, _, _ = C.time_two_phase(lambda: op(), lambda: None, 1, args["num_warmup"], args["num_experiments"])
    op.check()
    print(f"tcgen05  {m}x{n}x{k}: {total2 * 1e3:.1f} us = {2.0 * m * n * k / total2 / 1e9:.1f} TFLOPS "
          f"({100 * total / total2:.0f}% of cuBLAS)")


if __name__ == "__main__":
    main()
