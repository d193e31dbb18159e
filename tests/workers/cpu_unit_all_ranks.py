"""Worker run as N CPU ranks: the reference's unit-test semantics — every rank applies the primitive to EVERY
rank including itself, then a barrier and an exact comparison (tests/unittests/test_*.py)."""
import sys

import torch

import iris_b200 as iris


def main():
    ctx = iris.iris(1 << 20, backend="cpu")
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    for dtype in (torch.int8, torch.int32, torch.int64, torch.float32):
        for block in (1, 8, 16, 32):
            data = ctx.ones(block, dtype=dtype)
            res = ctx.zeros(block, dtype=dtype)
            ctx.barrier()
            iris.load(ctx, data, res, block=block)            # sum over ranks of ones
            assert torch.equal(res, torch.full((block,), world, dtype=dtype)), ("load", dtype, block)
            tmp = ctx.zeros(block, dtype=dtype)
            res2 = ctx.zeros(block, dtype=dtype)
            iris.get(ctx, data, tmp, res2, block=block)
            assert torch.equal(res2, torch.full((block,), world, dtype=dtype)), ("get", dtype, block)
            dst = ctx.zeros(block, dtype=dtype)
            ctx.barrier()
            iris.store(ctx, dst, 1, block=block)              # everyone writes 1 everywhere
            ctx.barrier()
            assert torch.equal(dst, torch.ones(block, dtype=dtype)), ("store", dtype, block)
            dst2 = ctx.zeros(block, dtype=dtype)
            ctx.barrier()
            iris.put(ctx, data, dst2, block=block)
            ctx.barrier()
            assert torch.equal(dst2, torch.ones(block, dtype=dtype)), ("put", dtype, block)
    for dtype in (torch.int32, torch.int64, torch.float32):
        for sem in ("relaxed", "acquire", "release", "acq_rel"):
            acc = ctx.zeros(16, dtype=dtype)
            ctx.barrier()
            iris.atomic_add(ctx, acc, 1, sem=sem, scope="sys", block=16)
            ctx.barrier()
            assert torch.equal(acc, torch.full((16,), world, dtype=dtype)), ("atomic_add", dtype, sem)
            x = ctx.zeros(1, dtype=dtype)
            ctx.barrier()
            iris.atomic_xchg(ctx, x, world, sem=sem, scope="sys", block=1)
            ctx.barrier()
            assert int(x[0]) == world, ("atomic_xchg", dtype, sem)
    for dtype in (torch.int16, torch.int32, torch.int64):
        f = ctx.zeros(1, dtype=dtype)
        ctx.barrier()
        iris.atomic_cas(ctx, f, 0, world, sem="acq_rel", scope="sys", block=1)
        ctx.barrier()
        assert int(f[0]) == world, ("atomic_cas", dtype)
    ctx.barrier()
    ctx.close()
    print(f"rank {rank}: OK")


if __name__ == "__main__":
    main()
    sys.exit(0)
