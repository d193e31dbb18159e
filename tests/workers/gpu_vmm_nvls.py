"""Worker run as one process per GPU with heap_mode="vmm": file-descriptor exchange, contiguous mapping of all
heaps, remote access through it and — when IRIS_NVLS=1 and the machine offers it — multicast stores and
switch-side all-reduce, each checked exactly or against PyTorch."""
import os
import sys

import torch

import iris_b200 as iris
from iris_b200.ops import nvls, p2p


def main():
    ctx = iris.iris(256 << 20, heap_mode="vmm")
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    hb = [int(x) for x in ctx.get_heap_bases().cpu().tolist()]
    stride = hb[1] - hb[0]
    assert all(hb[r] == hb[0] + r * stride for r in range(world)), "heaps are not contiguous in the address space"
    buf = ctx.zeros(4096, dtype=torch.float32)
    ctx.barrier()
    iris.store(ctx, buf, float(rank + 1), target=(rank + 1) % world, block=256)
    ctx.barrier()
    assert torch.equal(buf, torch.full_like(buf, float((rank - 1) % world + 1)))
    acc = ctx.zeros(64, dtype=torch.int32)
    ctx.barrier()
    iris.atomic_add(ctx, acc, 1, sem="relaxed", scope="sys", block=64)
    ctx.barrier()
    assert torch.equal(acc, torch.full_like(acc, world))
    msg = f"rank {rank}: VMM OK"
    if os.environ.get("IRIS_NVLS") == "1":
        if not nvls.available(ctx):
            msg += " (NVLS not available on this machine)"
        else:
            words = ctx.zeros(1 << 18, dtype=torch.int32)
            ctx.barrier()
            if rank == 0:
                nvls.all_store(ctx, words)
            ctx.barrier()
            assert torch.equal(words, torch.arange(words.numel(), dtype=torch.int32, device=dev)), "multimem.st"
            ar = nvls.AllReduce(ctx)
            x = ctx.zeros(1 << 20, dtype=torch.bfloat16)
            for it in range(3):
                g = torch.Generator(device=dev).manual_seed(100 + it)
                parts = [torch.randn(x.numel(), generator=g, device=dev).to(torch.bfloat16) for _ in range(world)]
                x.copy_(parts[rank])
                ctx.barrier()
                ar(x)
                ctx.barrier()
                ctx.check_status()
                ref = sum(p.float() for p in parts)
                assert (x.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item(), "multimem.ld_reduce"
            msg += " + NVLS OK"
    ctx.barrier()
    ctx.close()
    print(msg, flush=True)


if __name__ == "__main__":
    main()
    sys.exit(0)
