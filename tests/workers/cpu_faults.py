"""Worker for host-side failure tests on CPU ranks.  argv[1] selects the scenario."""
import os
import sys
import time

import torch

import iris_b200 as iris
from iris_b200 import _native
from iris_b200.parallel.bootstrap import BootstrapError


def main():
    scenario = sys.argv[1]
    rank = int(os.environ["RANK"])
    if scenario == "heap_size_mismatch":
        try:
            iris.iris((1 << 20) + (4096 if rank == 1 else 0), backend="cpu")
        except ValueError as e:
            print(f"rank {rank}: ValueError {e}")
            return 0
        return 1
    if scenario == "divergent_allocation":
        # debug heap: rank 1 allocates one buffer more than the others; the next barrier names the divergence
        ctx = iris.iris(1 << 20, backend="cpu", debug_heap=True)
        ctx.zeros(256, dtype=torch.float32)
        if rank == 1:
            ctx.zeros(8, dtype=torch.int32)
        try:
            ctx.barrier()
        except iris.context.IrisDivergenceError as e:
            print(f"rank {rank}: IrisDivergenceError {e}")
            return 0
        return 1
    if scenario == "remote_overrun":
        # debug heap: rank 0 writes 16 bytes past the end of a 1000-byte buffer of rank 1; rank 1's barrier says which
        import ctypes
        ctx = iris.iris(1 << 20, backend="cpu", debug_heap=True)
        first = ctx.zeros(100, dtype=torch.int32)
        buf = ctx.zeros(1000, dtype=torch.uint8)
        ctx.barrier()
        if rank == 0:
            peer = iris.translate(buf.data_ptr(), 0, 1, ctx.get_heap_bases().tolist())
            ctypes.memset(peer + 1008, 0x11, 16)
        ctx.comm.barrier()          # plain host barrier: the write has happened, nothing checked yet
        try:
            ctx.barrier()
        except iris.context.IrisHeapCorruption as e:   # every rank learns of it; the owner knows the details
            print(f"rank {rank}: IrisHeapCorruption {e}")
            return 0
        return 1
    ctx = iris.iris(1 << 20, backend="cpu")
    if scenario == "missing_rank_at_barrier":
        # rank 1 never joins the barrier: the others must get an error within the time limit, not hang
        if rank == 1:
            time.sleep(6)
            return 0
        t0 = time.time()
        try:
            ctx.barrier(timeout_s=2.0)
        except BootstrapError as e:
            print(f"rank {rank}: BootstrapError after {time.time() - t0:.1f}s")
            return 0
        return 1
    if scenario == "rank_dies":
        # rank 1 dies (no clean-up, no goodbye) after the first step; the others learn of it at their next barrier
        ctx.barrier()
        if rank == 1:
            os._exit(17)
        t0 = time.time()
        try:
            ctx.barrier(timeout_s=3.0)
        except BootstrapError:
            print(f"rank {rank}: peer loss detected after {time.time() - t0:.1f}s")
            return 0
        return 1
    if scenario == "heap_exhaustion":
        # the same allocation fails on every rank, with MemoryError and without moving the heap top
        big = ctx.zeros(200_000, dtype=torch.float32)
        top = ctx.mark()
        try:
            ctx.zeros(100_000, dtype=torch.float32)
        except MemoryError as e:
            assert ctx.mark() == top and str(e) == "Heap out of memory"
            small = ctx.zeros(1000, dtype=torch.float32)   # what still fits is still served, symmetrically
            ctx.barrier()
            print(f"rank {rank}: MemoryError, then {small.numel()} elements at offset {ctx.offset_of(small)}")
            return 0
        return 1
    if scenario == "flag_never_set":
        # consumer waits on a flag nothing sets: bounded wait returns a time-out status, recorded in the block
        flag = ctx.zeros(1, dtype=torch.int32)
        import ctypes
        rc = _native.cpu().iris_cpu_wait_flag(ctypes.c_void_p(flag.data_ptr()), 1, 200000,
                                              ctypes.c_void_p(ctx.status_ptr()), rank)
        assert rc == 1, rc
        try:
            ctx.check_status()
        except iris.IrisTimeoutError as e:
            print(f"rank {rank}: IrisTimeoutError {e}")
            ctx.barrier()
            return 0
        return 1
    if scenario == "message_passing":
        # producer = rank 0, consumer = rank 1; 4 chunks guarded by flags with release/acquire ordering
        import ctypes
        nchunks, chunk = 4, 1 << 14
        src = ctx.zeros(nchunks * chunk // 4, dtype=torch.float32)
        dst = ctx.zeros(nchunks * chunk // 4, dtype=torch.float32)
        flags = ctx.zeros(nchunks, dtype=torch.int32)
        lib = _native.cpu()
        hb = ctypes.c_void_p(ctx.get_heap_bases().data_ptr())
        ctx.barrier()
        for epoch in (1, 2):
            if rank == 0:
                src.copy_(torch.arange(src.numel(), dtype=torch.float32) + epoch)
                for c in range(nchunks):
                    lib.iris_cpu_mp_produce(ctypes.c_void_p(src.data_ptr() + c * chunk),
                                            ctypes.c_void_p(dst.data_ptr() + c * chunk), chunk,
                                            ctypes.c_void_p(flags.data_ptr() + 4 * c), epoch, hb, 0, 1)
            elif rank == 1:
                for c in range(nchunks):
                    rc = lib.iris_cpu_wait_flag(ctypes.c_void_p(flags.data_ptr() + 4 * c), epoch, 1 << 34,
                                                ctypes.c_void_p(ctx.status_ptr()), rank)
                    assert rc == 0
                    lo, hi = c * chunk // 4, (c + 1) * chunk // 4
                    expect = torch.arange(lo, hi, dtype=torch.float32) + epoch
                    assert torch.equal(dst[lo:hi], expect), (epoch, c)
            ctx.barrier()
        print(f"rank {rank}: OK")
        return 0
    return 2


if __name__ == "__main__":
    sys.exit(main())
