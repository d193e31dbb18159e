"""Worker run as 2+ CPU ranks: symmetric heap of 2^20 bytes per rank; fp32 buffer of 4096 elements, block 1024,
filled from seed 0 with N(0,1).  Rank 0 stores 1.0 into rank 1's buffer through heap-base translation, then
atomic_add(+rank), atomic_xchg and a load round trip, then barrier; all results are checked element-exact."""
import sys

import torch

import iris_b200 as iris


def main():
    ctx = iris.iris(1 << 20, backend="cpu")
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    assert world >= 2
    if "--expect-bootstrap" in sys.argv:  # the control plane the test asked for is the one in use
        want = sys.argv[sys.argv.index("--expect-bootstrap") + 1]
        assert type(ctx.comm).__name__ == want, type(ctx.comm).__name__
    n, block = 4096, 1024
    torch.manual_seed(0)
    buf = ctx.randn(n, dtype=torch.float32)
    init = buf.clone()
    counter = ctx.zeros(n, dtype=torch.int32)
    slot = ctx.zeros(n, dtype=torch.int32)
    old = ctx.zeros(n, dtype=torch.int32)
    back = ctx.zeros(n, dtype=torch.float32)
    hb = ctx.get_heap_bases()
    assert hb.numel() == world and int(hb[rank]) == ctx.heap_base()
    ctx.barrier()

    # 1. rank 0 stores 1.0 into rank 1's buffer
    if rank == 0:
        iris.store(ctx, buf, 1.0, target=1, block=block)
    ctx.barrier()
    if rank == 1:
        assert torch.equal(buf, torch.ones(n)), "remote store did not land"
    else:
        assert torch.equal(buf, init), "a rank other than 1 was modified"

    # 2. every rank adds +rank to rank 0's counter
    iris.atomic_add(ctx, counter, rank, target=0, sem="relaxed", scope="sys", block=block)
    ctx.barrier()
    if rank == 0:
        assert torch.equal(counter, torch.full((n,), sum(range(world)), dtype=torch.int32))

    # 3. rank 1 exchanges 42 into rank 0's slot and gets the previous value (0)
    if rank == 1:
        iris.atomic_xchg(ctx, slot, 42, old=old, target=0, sem="acq_rel", scope="sys", block=block)
        assert int(old.abs().sum()) == 0
    ctx.barrier()
    if rank == 0:
        assert torch.equal(slot, torch.full((n,), 42, dtype=torch.int32))

    # 4. load round trip: rank 0 reads rank 1's buffer (all ones now)
    if rank == 0:
        iris.load(ctx, buf, back, target=1, block=block)
        assert torch.equal(back, torch.ones(n))
    ctx.barrier()

    # 5. broadcast of a scalar from the last rank
    v = ctx.broadcast(float(rank) + 0.5, world - 1)
    assert v == world - 0.5
    ctx.barrier()
    ctx.close()
    print(f"rank {rank}: OK")


if __name__ == "__main__":
    main()
    sys.exit(0)
