"""Worker for the failure-detection test on GPUs: two steps of a fused GEMM + all-scatter; after the first step rank 1
leaves (between steps, with none of its kernels in flight, and without tearing anything down that peers map).  The
others learn of it on the host — their next barrier times out — BEFORE launching anything that would wait for the
missing rank, and finish cleanly.  No GPU wait ever runs out, no process is killed."""
import os
import sys

import torch

import iris_b200 as iris
from iris_b200.ops import gemm as G
from iris_b200.parallel.bootstrap import BootstrapError


def main():
    ctx = iris.iris(128 << 20)
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    g = torch.Generator(device=dev).manual_seed(1)
    a = torch.randn((512, 256), generator=g, device=dev).to(torch.bfloat16)
    bt = (torch.randn((256 * world, 256), generator=g, device=dev) * 0.05).to(torch.bfloat16)
    op = G.gemm_all_scatter(ctx, [a], [bt[rank * 256:(rank + 1) * 256].contiguous()])
    ctx.barrier()
    c = op()[0]
    ctx.barrier()
    op.check()
    ref = a.float() @ bt.float().t()
    assert (c.float() - ref).abs().max().item() <= 2 ** -6 * ref.abs().max().item()
    if rank == 1:
        torch.cuda.synchronize()
        print("rank 1: leaving after step 1", flush=True)
        os._exit(0)  # no further collective, no teardown that peers could observe half-done
    try:
        ctx.barrier(timeout_s=3.0)   # step 2 would start here
    except BootstrapError:
        torch.cuda.synchronize()
        print(f"rank {rank}: peer missing, step 2 not launched", flush=True)
        os._exit(0)
    print(f"rank {rank}: barrier passed although a rank left", flush=True)
    sys.exit(1)


if __name__ == "__main__":
    main()
