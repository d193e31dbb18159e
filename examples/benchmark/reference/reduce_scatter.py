#!/usr/bin/env python
"""Unfused baseline: cuBLAS GEMM on the K shard, then NCCL reduce-scatter of the partial over column blocks
(``examples/benchmark/reference/reduce_scatter.py:105-131`` of the reference)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _common as C  # noqa: E402
from _common import dist, torch  # noqa: E402


def main():
    args = C.parse_args("cuBLAS GEMM + NCCL reduce-scatter")
    rank, world, dev = C.init()
    m, n, k = args["m"], args["n"], args["k"]
    dt = C.dtype_of(args["datatype"])
    gen = torch.Generator(device=dev).manual_seed(3)
    A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(dt)
    Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(dt)
    ks, nl = k // world, n // world
    a_local = A[:, rank * ks:(rank + 1) * ks].contiguous()
    # B columns regrouped so that the partial comes out as [world, m, n/world]: block r is rank r's share
    b_blocks = Bt[:, rank * ks:(rank + 1) * ks].contiguous().view(world, nl, ks)
    stacked = torch.empty((world, m, nl), dtype=dt, device=dev)
    out = torch.empty((m, nl), dtype=dt, device=dev)

    def gemm():
        torch.matmul(a_local, b_blocks.transpose(1, 2), out=stacked)

    def comm():
        if world > 1:
            dist.reduce_scatter_tensor(out, stacked)
        else:
            out.copy_(stacked[0])
    ok = None
    if args["validate"]:
        gemm(); comm(); torch.cuda.synchronize()
        ref = A[:512, :ks * world].float() @ Bt[rank * nl:(rank + 1) * nl, :ks * world].float().t()
        ok = bool((out[:512].float() - ref).abs().max() <= (2 + world) * 2 ** -8 * ref.abs().max())
    total, g, cm = C.time_two_phase(gemm, comm, world, args["num_warmup"], args["num_experiments"])
    C.report(rank, args, "reduce_scatter", m, n, k, total, g, cm, ok)
    C.finish(world)


if __name__ == "__main__":
    main()
