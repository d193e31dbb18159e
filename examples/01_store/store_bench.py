#!/usr/bin/env python
"""Pairwise remote-STORE bandwidth: rank ``src`` writes the 32-bit word index into ``dst``'s buffer
(``examples/01_store/store_bench.py:20-46,88-166`` of the reference).  ``--validate`` checks the landed pattern."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import dtype_from_str, iris, pair_matrix, torch  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402


def parse_args():
    ap = argparse.ArgumentParser(description="Remote store bandwidth", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="fp16", choices=["int8", "fp16", "bf16", "fp32"])
    ap.add_argument("-z", "--buffer_size", type=int, default=1 << 28, help="bytes")
    ap.add_argument("-b", "--block_size", type=int, default=512)
    ap.add_argument("-g", "--grid", type=int, default=0)
    ap.add_argument("-v", "--verbose", action="store_true")
    ap.add_argument("-d", "--validate", action="store_true")
    ap.add_argument("-p", "--heap_size", type=int, default=1 << 30)
    ap.add_argument("-o", "--output_file", default="")
    ap.add_argument("-n", "--num_experiments", type=int, default=10)
    ap.add_argument("-w", "--num_warmup", type=int, default=1)
    return vars(ap.parse_args())


def main():
    args = parse_args()
    dtype_from_str(args["datatype"])  # the kernel moves 16-byte vectors; the datatype only names the run
    ctx = iris.iris(args["heap_size"])
    buf = ctx.zeros(args["buffer_size"] // 4, dtype=torch.int32)
    grid = args["grid"] or None

    def make_run(src, dst):
        return lambda: p2p.store(ctx, buf, target=dst, grid=grid, block=args["block_size"])

    pair_matrix(ctx, args, make_run, "Unidirectional STORE bandwidth GiB/s [Remote write]", args["buffer_size"])
    if args["validate"]:
        ok = torch.equal(buf, torch.arange(buf.numel(), dtype=torch.int32, device=buf.device))
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}.")
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
