#!/usr/bin/env python
"""ALL-LOAD: every rank simultaneously reads the same slice from all ranks, sums it and stores the sum locally;
swept over buffer sizes (``examples/02_all_load/all_load_bench.py:41-86,130-231,323-346`` of the reference).
Bytes counted per rank: (active - 1) * buffer, the store-only time is subtracted, GiB/s per GPU is reported."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import GIB, dtype_from_str, iris, time_kernel_ms, torch, write_json  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402
from iris_b200.utils.bench import reduce_ranks  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser(description="All-load bandwidth sweep", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="fp16", choices=["fp16", "bf16", "fp32"])
    ap.add_argument("-m", "--buffer_size_min", type=int, default=1 << 20)
    ap.add_argument("-M", "--buffer_size_max", type=int, default=1 << 30)
    ap.add_argument("-b", "--block_size", type=int, default=512)
    ap.add_argument("-g", "--grid", type=int, default=0)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-d", "--validate", action="store_true")
    ap.add_argument("-p", "--heap_size", type=int, default=(1 << 31) + (1 << 28))
    ap.add_argument("-x", "--num_experiments", type=int, default=20)
    ap.add_argument("-w", "--num_warmup", type=int, default=2)
    ap.add_argument("-a", "--active_ranks", type=int, default=8)
    ap.add_argument("-o", "--output_file", default="")
    return vars(ap.parse_args())


def main():
    args = parse_args()
    dtype = dtype_from_str(args["datatype"])
    ctx = iris.iris(args["heap_size"])
    world, rank = ctx.get_num_ranks(), ctx.get_rank()
    active = min(args["active_ranks"], world)
    es = torch.empty((), dtype=dtype).element_size()
    src = ctx.ones(args["buffer_size_max"] // es, dtype=dtype)
    out = ctx.zeros(args["buffer_size_max"] // es, dtype=dtype)
    grid = args["grid"] or None
    records = []
    size = args["buffer_size_min"]
    if rank == 0:
        print(f"ALL-LOAD, {active} active ranks, GiB/s per GPU (min / max over ranks)")
    while size <= args["buffer_size_max"]:
        on = rank < active
        run = lambda: p2p.all_load(ctx, src, out, active=active, nbytes=size, grid=grid, block=args["block_size"])
        sub = lambda: p2p.local_store(ctx, out, nbytes=size, grid=grid, block=args["block_size"])
        ms = time_kernel_ms(ctx, run, args["num_warmup"], args["num_experiments"], active=on)
        ms -= time_kernel_ms(ctx, sub, args["num_warmup"], args["num_experiments"], active=on)
        bw = (active - 1) * size / (ms * 1e-3) / GIB if on and ms > 0 and active > 1 else 0.0
        lo, hi = reduce_ranks(ctx, bw if on else 1e30, "min"), reduce_ranks(ctx, bw, "max")
        if rank == 0:
            print(f"{size / 2**20:10.2f} MiB  {lo:10.2f} {hi:10.2f}")
        records.append({"buffer_bytes": size, "gibps_min": lo, "gibps_max": hi, "active_ranks": active})
        if args["validate"] and on:
            run()  # the overhead kernel above wrote its own pattern into `out`: take the sum again
            torch.cuda.synchronize()
            assert float(out[: size // es].float().mean()) == float(active)
        size *= 2
    if rank == 0:
        write_json(args["output_file"], records)
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
