#!/usr/bin/env python
"""Producer / consumer message passing between two ranks with ``iris::put_block`` for the data and an int32
flag per chunk: the producer copies a chunk into the consumer's buffer and then raises the CONSUMER's flag with
release semantics; the consumer acquires its flag (bounded wait), doubles the data and writes it out.
Reference: ``examples/06_message_passing/message_passing_put.py:16-78,120-188`` (whose flags are local stores;
this is the protocol it intends).  Exactly two ranks.  ``--variant load_store`` uses per-element ``iris::load`` +
``iris::store`` instead of the block copy (``message_passing_load_store.py:15-90``)."""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import iris, time_kernel_ms, torch  # noqa: E402

from iris_b200.ops import p2p  # noqa: E402


def parse_args(default_variant="put"):
    ap = argparse.ArgumentParser(description="Message passing", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-t", "--datatype", default="fp32", choices=["fp32"])
    ap.add_argument("-s", "--buffer_size", type=int, default=8 << 18, help="elements (default: eight 1 MiB chunks)")
    ap.add_argument("-c", "--chunk_bytes", type=int, default=1 << 20)
    ap.add_argument("-b", "--block_size", type=int, default=512)
    ap.add_argument("-p", "--heap_size", type=int, default=1 << 30)
    ap.add_argument("-n", "--num_experiments", type=int, default=20)
    ap.add_argument("--variant", default=default_variant, choices=["put", "load_store"])
    ap.add_argument("--parts", type=int, default=None, help="slices (thread blocks at work) per chunk; default: from the sizes")
    ap.add_argument("--blocks", type=int, default=None,
                    help="thread blocks per side; fewer than chunks x parts makes the chunks land in order, so that "
                         "the consumer works on early chunks while later ones are on the link")
    return vars(ap.parse_args())


def main(default_variant="put"):
    args = parse_args(default_variant)
    ctx = iris.iris(args["heap_size"])
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    if world != 2:
        raise SystemExit("This example requires exactly two processes.")
    nchunks = max(1, args["buffer_size"] * 4 // args["chunk_bytes"])
    mp = p2p.MessagePassing(ctx, nchunks, args["chunk_bytes"], producer=0, consumer=1, timeout_ms=5000,
                            parts=args["parts"], blocks=args["blocks"])
    if rank == 0:
        mp.src.copy_(torch.arange(mp.src.numel(), device=mp.src.device, dtype=torch.float32) % 4096)
    use_put = args["variant"] == "put"
    ms = time_kernel_ms(ctx, lambda: mp.run(use_put=use_put, block=args["block_size"]), 2, args["num_experiments"])
    ctx.check_status()
    if rank == 1:
        want = 2 * (torch.arange(mp.src.numel(), device=mp.out.device, dtype=torch.float32) % 4096)
        ok = torch.equal(mp.out, want)
        gbs = nchunks * args["chunk_bytes"] / (ms * 1e-3) / 1e9
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}; consumer side {ms * 1e3:.1f} us per hand-off "
                f"of {nchunks} x {args['chunk_bytes']} B = {gbs:.1f} GB/s")
        if not ok:
            raise SystemExit(1)
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
