#!/usr/bin/env python
"""Pairwise remote ATOMIC_XCHG bandwidth (int32, relaxed, system scope; the old values are stored locally)
(``examples/05_atomic_xchg/atomic_xchg_bench.py:20-44`` of the reference)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import iris, pair_matrix, torch  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser(description="Remote atomic-exchange bandwidth", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="int32", choices=["int32"])
    ap.add_argument("-z", "--buffer_size", type=int, default=1 << 26, help="bytes")
    ap.add_argument("-b", "--block_size", type=int, default=512)
    ap.add_argument("-g", "--grid", type=int, default=0)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-d", "--validate", action="store_true")
    ap.add_argument("-p", "--heap_size", type=int, default=1 << 30)
    ap.add_argument("-o", "--output_file", default="")
    ap.add_argument("-x", "--num_experiments", type=int, default=16)
    ap.add_argument("-w", "--num_warmup", type=int, default=4)
    return vars(ap.parse_args())


def main():
    args = parse_args()
    ctx = iris.iris(args["heap_size"])
    buf = ctx.zeros(args["buffer_size"] // 4, dtype=torch.int32)
    old = ctx.zeros(args["buffer_size"] // 4, dtype=torch.int32)
    grid = args["grid"] or None

    def make_run(src, dst):
        return lambda: p2p.atomic_xchg_i32(ctx, buf, old, target=dst, grid=grid, block=args["block_size"])

    pair_matrix(ctx, args, make_run, "Unidirectional ATOMIC_XCHG bandwidth GiB/s [Remote atomic]", args["buffer_size"])
    if args["validate"]:
        ok = torch.equal(buf, torch.ones_like(buf))
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}.")
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
