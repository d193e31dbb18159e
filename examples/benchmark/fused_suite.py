#!/usr/bin/env python
"""One launch that measures every headline number of the repository on N ranks:

* P2P RMA: remote load / store between rank 0 and rank 1 from 4 KB to 1 GB, all-load / all-store plateaus,
  remote atomic add (fp32) and exchange (int32);
* GEMM + all-scatter on A[8192, 4096] x B[4096, 14336];
* GEMM + all-reduce (atomic, one-shot, two-shot, push two-shot, and the automatic choice) on K = 11008, N = 4096 for
  M in {1, 128, 1024, 8192};
* GEMM + reduce-scatter on M = 16384, N = 4096, K in {4096, 11008} (the decoder's row-parallel projections);

each fused kernel next to cuBLAS + NCCL on the same operands, device-timed, maximum over ranks, with the roofline
fraction.  Writes one JSON document (rank 0).  The reference spreads these over separate scripts and SLURM jobs
(``examples/benchmark/bench_all_shapes.py``, ``examples/benchmark/reference/*.py``).

    python -m iris_b200.launch -np 8 examples/benchmark/fused_suite.py --out results/suite_w8.json
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import GIB, device_barrier, iris, reduce_ranks, time_kernel_ms, torch  # noqa: E402

import torch.distributed as dist  # noqa: E402

from iris_b200.ops import gemm as G, p2p  # noqa: E402
from iris_b200.utils import roofline  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--out", default="")
    ap.add_argument("--reps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--skip_p2p", action="store_true")
    ap.add_argument("--skip_gemm", action="store_true")
    ap.add_argument("--max_p2p_bytes", type=int, default=1 << 30)
    ap.add_argument("--heap_mode", default=None, choices=["ipc", "vmm"],
                    help="vmm + IRIS_NVLS=1 in the environment binds the heap to an NVLS multicast object")
    args = ap.parse_args()
    ctx = iris.iris((3 << 30) + (1 << 29), heap_mode=args.heap_mode)
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    device_barrier(ctx)  # allocated first, so that it survives the heap rewinds below
    base = ctx.mark()
    peaks = roofline.load_peaks()
    res = {"heap_mode": ctx.heap_mode, "nvls": bool(ctx.mc_base), "world": world, "peaks": peaks.__dict__, "p2p": {}, "gemm": []}
    W, R = args.warmup, args.reps

    def log(msg):
        if rank == 0:
            print(msg, flush=True)

    # ------------------------------------------------------------------ P2P
    if not args.skip_p2p and world >= 2:
        big = ctx.zeros(args.max_p2p_bytes // 4, dtype=torch.int32)
        loc = ctx.zeros(args.max_p2p_bytes // 4, dtype=torch.int32)
        sweep = []
        size = 4096
        while size <= args.max_p2p_bytes:
            row = {"bytes": size}
            for name, fn in (("load", lambda: p2p.load(ctx, big, loc, target=1, nbytes=size)),
                             ("store", lambda: p2p.store(ctx, big, target=1, nbytes=size))):
                ms = time_kernel_ms(ctx, fn, 2, 10, active=(rank == 0), busy=True)
                row[name + "_gbs"] = ctx.broadcast(size / (ms * 1e-3) / 1e9 if rank == 0 and ms > 0 else 0.0, 0)
            sweep.append(row)
            log(f"p2p 0->1 {size:>11d} B  load {row['load_gbs']:8.1f} GB/s  store {row['store_gbs']:8.1f} GB/s")
            size *= 4 if size < (1 << 20) else 2
        res["p2p"]["pair_sweep"] = sweep
        nb = min(args.max_p2p_bytes, 1 << 28)
        f32 = big.view(torch.float32)
        for name, fn, moved in (
                ("all_load", lambda: p2p.all_load(ctx, f32, loc.view(torch.float32), nbytes=nb), (world - 1) * nb),
                ("all_store", lambda: p2p.all_store(ctx, big, nbytes=nb), (world - 1) * nb)):
            ms = time_kernel_ms(ctx, fn, 2, 10)
            bw = moved / (ms * 1e-3) / 1e9
            lo, hi = reduce_ranks(ctx, bw, "min"), reduce_ranks(ctx, bw, "max")
            res["p2p"][name] = {"bytes_per_peer": nb, "gbs_per_gpu_min": lo, "gbs_per_gpu_max": hi}
            log(f"{name}: {lo:.1f} .. {hi:.1f} GB/s per GPU ({nb >> 20} MiB per peer)")
        na = 1 << 24
        for name, fn in (("atomic_add_f32", lambda: p2p.atomic_add_f32(ctx, f32, target=1, n=na)),
                         ("atomic_add_f32_v4", lambda: p2p.atomic_add_f32(ctx, f32, target=1, n=na, vec4=True)),
                         ("atomic_xchg_i32", lambda: p2p.atomic_xchg_i32(ctx, big, loc, target=1, n=na))):
            ms = time_kernel_ms(ctx, fn, 2, 10, active=(rank == 0))
            bw = ctx.broadcast(na * 4 / (ms * 1e-3) / 1e9 if rank == 0 and ms > 0 else 0.0, 0)
            res["p2p"][name] = {"elements": na, "gbs": bw}
            log(f"{name} 0->1: {bw:.1f} GB/s")
        # producer / consumer hand-off of 1 MB chunks guarded by release / acquire flags (rank 0 -> rank 1)
        for nchunks in (8, 64):
            mp = p2p.MessagePassing(ctx, nchunks=nchunks, chunk_bytes=1 << 20, producer=0, consumer=1, timeout_ms=5000)
            ms = time_kernel_ms(ctx, lambda: mp.run(), 2, 10, busy=True)   # every rank launches its side (or nothing)
            us = ctx.broadcast(ms * 1e3 if rank == 1 else 0.0, 1)
            gbs = nchunks * (1 << 20) / (us * 1e-6) / 1e9 if us > 0 else 0.0
            ctx.check_status()
            res["p2p"][f"message_passing_{nchunks}x1MB"] = {"us_per_handoff": us, "gbs": gbs, "blocks_per_chunk": mp.parts}
            log(f"message passing {nchunks} x 1 MB, {mp.parts} blocks per chunk: {us:.1f} us per hand-off ({gbs:.0f} GB/s)")
        ctx.reset(base)

    # ------------------------------------------------------------------ fused GEMMs
    def bench_pair(label, op, unfused, flops, roof):
        ctx.barrier()
        op()
        ctx.barrier()
        op.check()
        ms = reduce_ranks(ctx, time_kernel_ms(ctx, lambda: op(), W, R, align=True), "max")
        op.check()
        bms = reduce_ranks(ctx, time_kernel_ms(ctx, unfused, W, R, align=True), "max")
        rec = dict(label, world=world, fused_us=ms * 1e3, fused_tflops=flops / (ms * 1e-3) / 1e12,
                   baseline_us=bms * 1e3, speedup=bms / ms, roofline_us=roof["target_us"], bound=roof["bound"],
                   roofline_fraction=roof["target_us"] / (ms * 1e3), cta_group=op.cta_group, ctas=op.ctas_per_rank)
        res["gemm"].append(rec)
        log(f"{label}{' [nvls]' if getattr(op, 'nvls', False) else ''}: fused {rec['fused_us']:.1f} us ({rec['fused_tflops']:.0f} TF) | cuBLAS+NCCL {rec['baseline_us']:.1f} us "
            f"| x{rec['speedup']:.2f} | roofline {roof['target_us']:.0f} us ({roof['bound']}) -> {100 * rec['roofline_fraction']:.0f}%")

    if not args.skip_gemm:
        # config 3: GEMM + all-scatter
        m, n, k = 8192, 14336, 4096
        if n % world == 0:
            gen = torch.Generator(device=dev).manual_seed(2)
            A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            nl = n // world
            btl = Bt[rank * nl:(rank + 1) * nl].contiguous()
            del Bt
            op = G.gemm_all_scatter(ctx, [A], [btl])
            c_part = torch.empty((m, nl), dtype=torch.bfloat16, device=dev)
            gathered = torch.empty((world, m, nl), dtype=torch.bfloat16, device=dev)

            def unfused():
                torch.matmul(A, btl.t(), out=c_part)
                if world > 1:
                    dist.all_gather_into_tensor(gathered, c_part)
            bench_pair({"workload": "all_scatter", "m": m, "n": n, "k": k}, op, unfused, 2.0 * m * n * k,
                       roofline.all_scatter_roofline_us(m, n, k, world, peaks))
            ref = A[:256].float() @ btl.float().t()
            err = (op.out[0][:256, rank * nl:(rank + 1) * nl].float() - ref).abs().max().item()
            assert err <= 2 ** -6 * ref.abs().max().item(), f"all_scatter validation failed: {err}"
            op.close()
            del A, btl, c_part, gathered
            ctx.reset(base)
        # config 4: GEMM + all-reduce
        n, k = 4096, 11008
        if k % world == 0 and (k // world) % 8 == 0:
            ks = k // world
            gen = torch.Generator(device=dev).manual_seed(3)
            Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            for m in (8192, 1024, 128, 1):
                A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
                al, bl = A[:, rank * ks:(rank + 1) * ks], Bt[:, rank * ks:(rank + 1) * ks]
                c_part = torch.empty((m, n), dtype=torch.bfloat16, device=dev)

                def unfused():
                    torch.matmul(al, bl.t(), out=c_part)
                    if world > 1:
                        dist.all_reduce(c_part)
                ref = A[:128].float() @ Bt.float().t()
                for variant in ("atomic", "one_shot", "two_shot", "two_shot_push", "auto"):
                    if variant == "two_shot_push" and m % (world * 128):
                        continue
                    op = G.gemm_all_reduce(ctx, [al], [bl], variant=variant)
                    chosen = "atomic" if op.mode == "reduce" else ("two_shot_push" if op.bcast else op.mode)
                    label = {"workload": variant, "m": m, "n": n, "k": k, "tile": f"{128 * op.cta_group}x{op.bn}",
                             "ksplit": op.ksplit}
                    if variant == "auto":
                        label["chosen"] = chosen
                    bench_pair(label, op, unfused, 2.0 * m * n * k,
                               roofline.all_reduce_roofline_us(m, n, k, world, peaks,
                                                               "two_shot" if chosen.startswith("two_shot") else "one_shot"))
                    err = (op.out[0][:128].float() - ref).abs().max().item()
                    tol = (2 + world * op.ksplit) * 2 ** -8 * ref.abs().max().item() + 1e-3
                    assert err <= tol, f"{variant} m={m}: err {err}"
                    op.close()
                    ctx.reset(base)
                del A, c_part
        # the row-parallel projections of the decoder stack as GEMM + reduce-scatter: 16384 tokens, N = 4096
        m, n = 16384, 4096
        for k in (4096, 11008):
            if k % world or (k // world) % 8 or m % (world * 256):
                continue
            ks = k // world
            gen = torch.Generator(device=dev).manual_seed(5)
            A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
            al, bl = A[:, rank * ks:(rank + 1) * ks], Bt[:, rank * ks:(rank + 1) * ks]
            c_part = torch.empty((m, n), dtype=torch.bfloat16, device=dev)
            c_kept = torch.empty((m // world, n), dtype=torch.bfloat16, device=dev)

            def unfused_rs():
                torch.matmul(al, bl.t(), out=c_part)
                if world > 1:
                    dist.reduce_scatter_tensor(c_kept, c_part)
            op = G.gemm_reduce_scatter(ctx, [al], [bl])
            bench_pair({"workload": "reduce_scatter", "m": m, "n": n, "k": k}, op, unfused_rs, 2.0 * m * n * k,
                       roofline.all_reduce_roofline_us(m, n, k, world, peaks, "reduce_scatter"))
            r0 = rank * (m // world)
            ref = A[r0:r0 + 128].float() @ Bt.float().t()
            err = (op.out[0][:128].float() - ref).abs().max().item()
            assert err <= (2 + world) * 2 ** -8 * ref.abs().max().item() + 1e-3, f"reduce_scatter k={k}: err {err}"
            op.close()
            del A, Bt, c_part, c_kept
            ctx.reset(base)
    if rank == 0 and args.out:
        os.makedirs(os.path.dirname(args.out) or ".", exist_ok=True)
        with open(args.out, "w") as f:
            json.dump(res, f, indent=2)
    ctx.barrier()
    ctx.close()


if __name__ == "__main__":
    main()
