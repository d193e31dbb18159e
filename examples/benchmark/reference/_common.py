"""Shared set-up of the unfused baselines: torch.distributed (NCCL) initialisation from the launcher's environment,
seeded operands, device timing with GEMM and collective timed separately, JSON output.

Role in the reference: the common parts of ``examples/benchmark/reference/all_gather.py:19-183``,
``all_reduce.py`` and ``reduce_scatter.py`` (torch.distributed "nccl" = RCCL there, NCCL here)."""
from __future__ import annotations

import argparse
import json
import os
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402


def parse_args(desc: str):
    ap = argparse.ArgumentParser(description=desc, formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-m", type=int, default=8192)
    ap.add_argument("-n", type=int, default=8192)
    ap.add_argument("-k", type=int, default=30720)
    ap.add_argument("-v", "--validate", action="store_true")
    ap.add_argument("-b", "--benchmark", action="store_true")
    ap.add_argument("-d", "--datatype", default="bf16", choices=["fp16", "fp32", "bf16"])
    ap.add_argument("-o", "--output_file", default="")
    ap.add_argument("--num_experiments", type=int, default=50)
    ap.add_argument("--num_warmup", type=int, default=10)
    return vars(ap.parse_args())


def init():
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29544")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, torch.device("cuda", local)


def dtype_of(name):
    return {"fp16": torch.float16, "fp32": torch.float32, "bf16": torch.bfloat16}[name]


def time_two_phase(gemm_fn, comm_fn, world, warmup, repeat):
    """Returns (total_ms, gemm_ms, comm_ms), each the max over ranks of the mean device time; GEMM and
    collective run back to back on one stream (no overlap by construction, as in the reference,
    examples/benchmark/reference/all_reduce.py:116-131)."""
    ev = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(repeat)]
    for i in range(-warmup, repeat):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        if i >= 0:
            ev[i][0].record()
        gemm_fn()
        if i >= 0:
            ev[i][1].record()
        comm_fn()
        if i >= 0:
            ev[i][2].record()
    torch.cuda.synchronize()
    g = sum(e[0].elapsed_time(e[1]) for e in ev) / repeat
    c = sum(e[1].elapsed_time(e[2]) for e in ev) / repeat
    t = torch.tensor([g + c, g, c], device="cuda", dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return tuple(float(x) for x in t)


def report(rank, args, algorithm, m, n, k, total, gemm, comm, success=None):
    if rank != 0:
        return
    tflops = 2.0 * m * n * k / (total * 1e-3) / 1e12
    rec = dict(args, algorithm=algorithm, ms=total, gemm_ms=gemm, communication_ms=comm, flops=tflops)
    if success is not None:
        rec["success"] = success
    print(f"{algorithm}: total {total * 1e3:.1f} us (GEMM {gemm * 1e3:.1f} + collective {comm * 1e3:.1f}) = "
          f"{tflops:.1f} TFLOPS", flush=True)
    if args["output_file"]:
        with open(args["output_file"], "w") as f:
            json.dump(rec, f, indent=2)


def finish(world):
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
