#!/usr/bin/env python
"""Pairwise remote ATOMIC_ADD bandwidth (relaxed, system scope, result unused), counting the bytes of the elements
updated (``examples/04_atomic_add/atomic_add_bench.py:20-41,85-164`` of the reference).  ``--datatype`` takes the
reference's fp16 (its default) / bf16 / fp32 plus int32 / int64; int8 is not offered: sm_100a has no 8-bit atomic."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import dtype_from_str, iris, pair_matrix, torch  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser(description="Remote atomic-add bandwidth", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="fp32", choices=["fp16", "bf16", "fp32", "int32", "int64"])
    ap.add_argument("-z", "--buffer_size", type=int, default=1 << 26, help="bytes")
    ap.add_argument("-b", "--block_size", type=int, default=512)
    ap.add_argument("-g", "--grid", type=int, default=0)
    ap.add_argument("--vec4", action="store_true", help="use 16-byte vector reductions")
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
    dtype = torch.int64 if args["datatype"] == "int64" else dtype_from_str(args["datatype"])
    buf = ctx.zeros(args["buffer_size"] // torch.empty((), dtype=dtype).element_size(), dtype=dtype)
    grid = args["grid"] or None
    if args["vec4"] and dtype != torch.float32:
        raise SystemExit("--vec4 (16-byte vector reductions) exists for fp32 only")

    def make_run(src, dst):
        if dtype == torch.float32:
            return lambda: p2p.atomic_add_f32(ctx, buf, target=dst, vec4=args["vec4"], grid=grid,
                                              block=args["block_size"])
        return lambda: p2p.atomic_add(ctx, buf, target=dst, grid=grid, block=args["block_size"])

    pair_matrix(ctx, args, make_run, "Unidirectional ATOMIC_ADD bandwidth GiB/s [Remote atomic]", args["buffer_size"])
    if args["validate"]:
        total = ctx.get_num_ranks() * (args["num_experiments"] + args["num_warmup"])
        ok = torch.equal(buf, torch.full_like(buf, total))
        ctx.log(f"Validation {'successful' if ok else 'FAILED'} (every element == {total}).")
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
