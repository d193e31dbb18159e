#!/usr/bin/env python
"""Pairwise remote-LOAD bandwidth: for every (src, dst) rank pair only rank ``src`` launches a kernel that reads
``dst``'s buffer over NVLink and writes it locally; the time of a local-store-only kernel is subtracted, as the
reference does (``examples/00_load/load_bench.py:103-193``).  Flags as the reference (``:78-100``) with B200-sized
defaults (256 MiB buffer) and one extra, ``--grid``, because the kernel is a persistent grid-stride loop.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import dtype_from_str, iris, pair_matrix, torch  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser(description="Remote load bandwidth", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="fp16", choices=["int8", "fp16", "bf16", "fp32"])
    ap.add_argument("-z", "--buffer_size", type=int, default=1 << 28, help="bytes")
    ap.add_argument("-b", "--block_size", type=int, default=512, help="threads per CTA")
    ap.add_argument("-g", "--grid", type=int, default=0, help="CTAs (0: 4 per SM)")
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-d", "--validate", action="store_true")
    ap.add_argument("-p", "--heap_size", type=int, default=1 << 30)
    ap.add_argument("-o", "--output_file", default="")
    ap.add_argument("-n", "--num_experiments", type=int, default=10)
    ap.add_argument("-w", "--num_warmup", type=int, default=1)
    ap.add_argument("--no_subtract", action="store_true", help="report raw kernel time (no local-store subtraction)")
    return vars(ap.parse_args())


def main():
    args = parse_args()
    dtype = dtype_from_str(args["datatype"])
    ctx = iris.iris(args["heap_size"])
    n = args["buffer_size"] // torch.empty((), dtype=dtype).element_size()
    src_buf = ctx.ones(n, dtype=dtype)
    dst_buf = ctx.zeros_like(src_buf)
    grid = args["grid"] or None

    def make_run(src, dst):
        return lambda: p2p.load(ctx, src_buf, dst_buf, target=dst, grid=grid, block=args["block_size"])

    sub = None if args["no_subtract"] else (lambda: p2p.local_store(ctx, dst_buf, grid=grid, block=args["block_size"]))
    pair_matrix(ctx, args, make_run, "Unidirectional LOAD bandwidth GiB/s [Remote read]", args["buffer_size"], sub)
    if args["validate"]:
        p2p.load(ctx, src_buf, dst_buf, target=(ctx.get_rank() + 1) % ctx.get_num_ranks(), grid=grid)
        ctx.barrier()
        ok = torch.equal(dst_buf, src_buf)
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}.")
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
