"""Timing and reporting helpers shared by the example scripts.

Role in the reference: the per-script copies of argument parsing, ``do_bench`` loops, bandwidth-matrix printing
and JSON output (``examples/00_load/load_bench.py:78-229`` and its siblings).  Here they exist once.

Run any example with ``python -m iris_b200.launch -np N examples/<dir>/<script>.py [flags]`` (or ``torchrun``).
"""
from __future__ import annotations

import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402

import iris_b200 as iris  # noqa: E402
from iris_b200.utils.bench import reduce_ranks  # noqa: E402

DTYPES = {"int8": torch.int8, "int32": torch.int32, "fp16": torch.float16, "bf16": torch.bfloat16,
          "fp32": torch.float32}
GIB = float(1 << 30)


def dtype_from_str(name: str) -> torch.dtype:
    if name not in DTYPES:
        raise SystemExit(f"Unknown datatype: {name}")
    return DTYPES[name]


_device_barriers = {}


def device_barrier(ctx):
    """The context's device-side barrier (created on first use: allocate it before taking a heap mark)."""
    from iris_b200.ops.p2p import DeviceBarrier
    if ctx.get_num_ranks() == 1:
        return None
    b = _device_barriers.get(id(ctx))
    if b is None:
        b = _device_barriers[id(ctx)] = DeviceBarrier(ctx)
    return b


def time_kernel_ms(ctx, fn, n_warmup: int, n_repeat: int, active: bool = True, align: bool = False,
                   busy: bool = False) -> float:
    """Mean device time of ``fn`` in ms on the ranks where ``active``; every rank takes part in the barriers
    (``iris/util.py:62-104``: barrier, then event / launch / event, every iteration).  With ``align`` a
    device-side barrier kernel runs on every rank right before the start event, so the ranks' streams start the
    timed launch together and host launch skew is not charged to a kernel that waits for its peers.  ``busy`` alone
    only keeps the GPU occupied while the host enqueues, so that a short kernel is not timed with launch latency."""
    dbar = device_barrier(ctx) if align else None
    e0 = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    e1 = [torch.cuda.Event(enable_timing=True) for _ in range(n_repeat)]
    for i in range(-n_warmup, n_repeat):
        ctx.barrier()
        if align or busy:
            # Keep the GPU busy while the host enqueues [barrier, event, launch, event]: otherwise a short kernel is
            # timed together with the host's launch latency.
            torch.cuda._sleep(300000)
        if dbar is not None:
            dbar()
        if active:
            if i >= 0:
                e0[i].record()
            fn()
            if i >= 0:
                e1[i].record()
    ctx.barrier()
    if not active:
        return 0.0
    return sum(a.elapsed_time(b) for a, b in zip(e0, e1)) / max(1, n_repeat)


def print_matrix(matrix, label: str) -> None:
    n = len(matrix)
    w = 10
    print(f"\n{label}")
    print(" SRC\\DST".ljust(w) + "".join(f"GPU {j:02d}".rjust(w) for j in range(n)))
    for i in range(n):
        print(f"GPU {i:02d}  ->".ljust(w) + "".join(f"{matrix[i][j]:.2f}".rjust(w) for j in range(n)))


def write_json(path: str, records) -> None:
    if not path:
        return
    d = os.path.dirname(path)
    if d:
        os.makedirs(d, exist_ok=True)
    with open(path, "w") as f:
        json.dump(records, f, indent=2)


def pair_matrix(ctx, args, make_run, label: str, bytes_moved: int, subtract=None):
    """Time ``make_run(src, dst)`` for every ordered pair of ranks; only rank ``src`` launches.  Returns the
    matrix in GiB/s (and prints it / writes JSON on rank 0)."""
    world, rank = ctx.get_num_ranks(), ctx.get_rank()
    matrix = [[0.0] * world for _ in range(world)]
    records = []
    for src in range(world):
        for dst in range(world):
            run = make_run(src, dst)
            ms = time_kernel_ms(ctx, run, args["num_warmup"], args["num_experiments"], active=(rank == src))
            if subtract is not None:
                ms -= time_kernel_ms(ctx, subtract, args["num_warmup"], args["num_experiments"], active=(rank == src))
            bw = bytes_moved / (ms * 1e-3) / GIB if rank == src and ms > 0 else 0.0
            bw = ctx.broadcast(bw, src)
            matrix[src][dst] = float(bw)
            records.append({"source_rank": src, "destination_rank": dst, "bandwidth_gibps": float(bw),
                            "bandwidth_gbps": float(bw) * GIB / 1e9, "bytes": bytes_moved})
            if args.get("verbose") and rank == 0:
                ctx.log(f"{src} -> {dst}: {bw:.2f} GiB/s")
    if rank == 0:
        print_matrix(matrix, label)
        write_json(args.get("output_file", ""), records)
    return matrix
