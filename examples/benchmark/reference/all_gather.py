#!/usr/bin/env python
"""Unfused baseline of GEMM + all-scatter: cuBLAS ``A @ B_local`` then NCCL all-gather of the column blocks
(``examples/benchmark/reference/all_gather.py:113-141`` of the reference, where the library is RCCL).  The gather
lands in a contiguous ``[world, m, n/world]`` buffer so the library collective is not handicapped by strided
outputs."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import _common as C  # noqa: E402
from _common import dist, torch  # noqa: E402


def main():
    args = C.parse_args("cuBLAS GEMM + NCCL all-gather")
    rank, world, dev = C.init()
    m, n, k = args["m"], args["n"], args["k"]
    dt = C.dtype_of(args["datatype"])
    gen = torch.Generator(device=dev).manual_seed(2)
    A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(dt)
    Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(dt)
    nl = n // world
    b_local = Bt[rank * nl:(rank + 1) * nl].contiguous().t()
    c_part = torch.empty((m, nl), dtype=dt, device=dev)
    gathered = torch.empty((world, m, nl), dtype=dt, device=dev)

    def gemm():
        torch.matmul(A, b_local, out=c_part)

    def comm():
        if world > 1:
            dist.all_gather_into_tensor(gathered, c_part)
        else:
            gathered[0].copy_(c_part)
    ok = None
    if args["validate"]:
        gemm(); comm(); torch.cuda.synchronize()
        full = gathered.permute(1, 0, 2).reshape(m, n)
        ref = A[:512].float() @ Bt.float().t()
        ok = bool((full[:512].float() - ref).abs().max() <= 2 ** -6 * ref.abs().max())
    total, g, c = C.time_two_phase(gemm, comm, world, args["num_warmup"], args["num_experiments"])
    C.report(rank, args, "all_gather", m, n, k, total, g, c, ok)
    C.finish(world)


if __name__ == "__main__":
    main()
