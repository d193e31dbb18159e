#!/usr/bin/env python
"""Unfused baseline of GEMM + all-reduce: cuBLAS ``A_local @ B_local`` on the K shard, then NCCL all-reduce of the
``[m, n]`` partial (``examples/benchmark/reference/all_reduce.py:109-137`` of the reference)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _common as C  # noqa: E402
from _common import dist, torch  # noqa: E402


def main():
    args = C.parse_args("cuBLAS GEMM + NCCL all-reduce")
    rank, world, dev = C.init()
    m, n, k = args["m"], args["n"], args["k"]
    dt = C.dtype_of(args["datatype"])
    gen = torch.Generator(device=dev).manual_seed(3)
    A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(dt)
    Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(dt)
    ks = k // world
    a_local = A[:, rank * ks:(rank + 1) * ks].contiguous()
    b_local = Bt[:, rank * ks:(rank + 1) * ks].contiguous().t()
    c = torch.empty((m, n), dtype=dt, device=dev)

    def gemm():
        torch.matmul(a_local, b_local, out=c)

    def comm():
        if world > 1:
            dist.all_reduce(c)
    ok = None
    if args["validate"]:
        gemm(); comm(); torch.cuda.synchronize()
        ref = A[:512, :ks * world].float() @ Bt[:, :ks * world].float().t()
        ok = bool((c[:512].float() - ref).abs().max() <= (2 + world) * 2 ** -8 * ref.abs().max())
    total, g, cm = C.time_two_phase(gemm, comm, world, args["num_warmup"], args["num_experiments"])
    C.report(rank, args, "all_reduce", m, n, k, total, g, cm, ok)
    C.finish(world)


if __name__ == "__main__":
    main()
