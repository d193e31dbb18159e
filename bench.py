#!/usr/bin/env python
"""Headline benchmark: fused GEMM + all-scatter on the named configuration.

    C[8192, 14336] = A[8192, 4096] . B[4096, 14336]     bf16, fp32 accumulation, N(0, 0.02), seed 2
    A replicated, B sharded column-wise over the N GPUs; every rank computes its column block with the
    tcgen05 kernel and pushes every finished tile into the C of all ranks over NVLink.

    python bench.py --gpus 1 --steps 20 --warmup 5
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 --master-port 29500 \
        bench.py --gpus 8 --steps 20 --warmup 5

Rank 0 prints ONE JSON line.

``value`` is the whole-job TFLOP/s (2 M N K / time, global M N K as the reference computes it,
``examples/07_gemm_all_scatter/benchmark.py:253-271``).  Every step has its own pair of CUDA events on the launching
stream (the reference times every iteration separately too, ``iris/util.py:62-104``); per step the maximum over
ranks is taken and ``ms_per_step`` is the median of those, with mean / min / max / p10 / p90 and the raw list beside
it.  Before the first timed launch the ranks' streams are aligned by a barrier kernel on the GPUs, so that host-side
skew is not charged to a kernel that waits for its peers; the clock sampler is started (and has delivered its first
sample) before that.

``e2e`` is the same product through the public API with, per step, the host-to-device copy of that step's input
from pinned memory and a device-to-host read of one row of the result.  On one GPU the whole A is copied; on N GPUs
every rank copies its own M / N rows and the kernel's all-gather prologue distributes them over NVLink while the
tiles whose rows are already present are computed.

``same_box_baseline`` is cuBLAS + NCCL on the same operands, timed the same way (kernel-only and end to end), and
``vs_baseline`` is our ``value`` divided by its TFLOP/s.  ``selfcheck`` (N >= 2, untimed) runs the other fused
collectives on small shapes against an fp32 product, three calls back to back, and reports error / tolerance.
``--impl reference`` reports why the reference (HIP / Triton-AMD only) cannot run on this machine.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

M, N, K = 8192, 14336, 4096
SEED = 2


def reference_arm():
    print(json.dumps({
        "impl": "reference",
        "unavailable": "ROCm/iris needs hipcc, libamdhip64 and Triton-AMD on MI300X; its offline install fails here "
                       "at 'hipcc not found' (setup.py build of the fine-grained allocator), so it cannot run on B200"}))
    return 0


def _stats(ms):
    s = sorted(ms)
    q = lambda f: s[min(len(s) - 1, int(f * len(s)))]  # noqa: E731
    return {"median": round(statistics.median(s), 4), "mean": round(statistics.fmean(s), 4), "min": round(s[0], 4),
            "max": round(s[-1], 4), "p10": round(q(0.10), 4), "p90": round(q(0.90), 4)}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=300)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-baseline", action="store_true", help="skip the untimed cuBLAS+NCCL comparison")
    ap.add_argument("--no-selfcheck", action="store_true", help="skip the small-shape check of the other collectives")
    ap.add_argument("--push-kind", default=None, choices=["tma", "tma_spread", "stores", "multimem"],
                    help="how finished tiles travel to the other ranks (default: the library's default)")
    ap.add_argument("--heap-mode", default=None, choices=["ipc", "vmm"],
                    help="vmm (with IRIS_NVLS=1) binds the heap to an NVLS multicast object; needed by multimem")
    args = ap.parse_args()
    if args.impl == "reference":
        return reference_arm()
    if args.warmup < 3:
        args.warmup = 3

    import torch
    import torch.distributed as dist

    import iris_b200 as iris
    from iris_b200.ops import gemm as G
    from iris_b200.ops.p2p import DeviceBarrier
    from iris_b200.utils.bench import ClockSampler

    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            print(json.dumps({"error": f"--gpus {args.gpus} needs torch.distributed.run with that many ranks"}))
            return 2
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group(backend="cpu:gloo,cuda:nccl", device_id=dev)

    n_local = N // world
    ms_rows = M // world
    # two C buffers (235 MB each: kernel-only and the two end-to-end plans share them in turn), two gathered A,
    # the self-check's small buffers, flags
    heap = 3 * (2 * M * N) + 2 * (2 * M * K) + (256 << 20)
    ctx = iris.iris(heap, heap_mode=args.heap_mode)
    dbar = DeviceBarrier(ctx) if world > 1 else None

    # synthetic data of the named shape: same seed on every rank -> identical A and B everywhere
    gen = torch.Generator(device=dev).manual_seed(SEED)
    a_dev = (torch.randn((M, K), generator=gen, device=dev) * 0.02).to(torch.bfloat16)
    bt_full = (torch.randn((N, K), generator=gen, device=dev) * 0.02).to(torch.bfloat16)  # B^T: [N, K], K-major
    bt_local = bt_full[rank * n_local:(rank + 1) * n_local].clone()
    peer = (rank + 1) % world
    bt_peer = bt_full[peer * n_local:(peer + 1) * n_local].clone() if world > 1 else None
    del bt_full
    a_host = a_dev.cpu().pin_memory()
    rows_host = [torch.empty((N,), dtype=torch.bfloat16).pin_memory() for _ in range(2)]

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
            torch.cuda.synchronize()

    def max_over_ranks(values):
        """Element-wise maximum over the ranks of a list of floats."""
        if world == 1:
            return list(values)
        t = torch.tensor(values, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return t.tolist()

    def validate(c, what):
        """This rank's own column block and the block pushed by the next rank, first and last rows, against fp32."""
        worst = 0.0
        for blk, bt in ((rank, bt_local), (peer, bt_peer)):
            if bt is None:
                continue
            for rows in (slice(0, 512), slice(M - 256, M)):
                ref = a_dev[rows].float() @ bt.float().t()
                got = c[rows, blk * n_local:(blk + 1) * n_local].float()
                err = (got - ref).abs().max().item()
                tol = 2.0 ** -7 * max(ref.abs().max().item(), 1e-6)
                if not err <= tol:
                    raise RuntimeError(f"{what}: rank {rank}, column block of rank {blk}, rows {rows.start}..: "
                                       f"max err {err} > {tol}")
                worst = max(worst, err / tol)
        return worst

    def timed_steps(fn, steps):
        """Per-step device time (ms, maximum over ranks) of `steps` back-to-back calls of fn."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
        barrier()
        torch.cuda._sleep(3_000_000)       # the device idles ~1.5 ms while the host enqueues ahead of it
        if dbar is not None:
            dbar()                         # the ranks' streams start the first step together
        for s, e in ev:
            s.record()
            fn()
            e.record()
        barrier()
        return max_over_ranks([s.elapsed_time(e) for s, e in ev])

    out = {}
    try:
        op = G.gemm_all_scatter(ctx, [a_dev], [bt_local], push_kind=args.push_kind)
        c = op.out[0]

        # ---- correctness of one call: own block and a block pushed by a peer ----
        op()
        barrier()
        op.check()
        validate(c, "kernel-only op")

        # ---- the other fused collectives on small shapes (untimed) ----
        selfcheck = None
        if world > 1 and not args.no_selfcheck:
            selfcheck = run_selfcheck(ctx, G, torch, dist, dev, rank, world, barrier)

        # ---- device-timed kernel-only measurement ----
        sampler = None
        if rank == 0:
            sampler = ClockSampler(local_rank, period_ms=10).start()
            sampler.wait_first_sample(10.0)
        for _ in range(args.warmup):
            op()
        launches0 = op.launches
        per_step = timed_steps(op, args.steps)
        launches = op.launches - launches0
        op.check()
        st = _stats(per_step)
        ms_step = st["median"]
        tflops = 2.0 * M * N * K / (ms_step * 1e-3) / 1e12

        # ---- end to end through the public API: H2D of this step's input, fused op, D2H of one row of C ----
        # Two buffer sets (and a plan on each) let the copy of step i+1 run on a side stream while step i computes.
        # The result row of step i is copied back asynchronously; the host waits for the row of step i-1 after it has
        # launched step i (a caller that consumes every result, one step behind, so that the device never idles
        # waiting for the host to launch).
        copy_stream = torch.cuda.Stream(device=dev)
        main_stream = torch.cuda.current_stream()
        ready = [torch.cuda.Event(), torch.cuda.Event()]
        consumed = [torch.cuda.Event(), torch.cuda.Event()]
        d2h_done = [torch.cuda.Event(), torch.cuda.Event()]
        if world == 1:
            a_bufs = [a_dev, torch.empty_like(a_dev)]
            ops = [op, G.gemm_all_scatter(ctx, [a_bufs[1]], [bt_local])]
            src_host, dst_dev = a_host, a_bufs
        else:
            # every rank copies its own rows; the all-gather prologue of the kernel fetches the rest over NVLink
            ops = [G.FusedGemm(ctx, None, [bt_local], "store", M=M, ag=True, store_all=True, c_cols=N,
                               col_off_per_rank=n_local, push_kind=args.push_kind) for _ in range(2)]
            src_host = a_host[rank * ms_rows:(rank + 1) * ms_rows]
            dst_dev = [o.a_full[0][rank * ms_rows:(rank + 1) * ms_rows] for o in ops]
        h2d_bytes = src_host.numel() * src_host.element_size()

        def e2e_steps(run, dst, n):
            for b in (0, 1):
                consumed[b].record(main_stream)

            def prefetch(i):
                b = i & 1
                with torch.cuda.stream(copy_stream):
                    copy_stream.wait_event(consumed[b])      # the step that read this buffer two steps ago is done
                    dst[b].copy_(src_host, non_blocking=True)
                    ready[b].record(copy_stream)
            prefetch(0)
            for i in range(n):
                b = i & 1
                if i + 1 < n:
                    prefetch(i + 1)
                main_stream.wait_event(ready[b])
                row = run(b)
                consumed[b].record(main_stream)
                rows_host[b].view(row.shape).copy_(row, non_blocking=True)
                d2h_done[b].record(main_stream)
                if i >= 1:
                    d2h_done[b ^ 1].synchronize()            # the row of step i-1 is on the host: the caller uses it
            d2h_done[(n - 1) & 1].synchronize()

        def time_e2e(run, dst):
            e2e_steps(run, dst, 4)
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            if dbar is not None:
                dbar()
            e0.record()
            e2e_steps(run, dst, args.steps)
            e1.record()
            barrier()
            return max_over_ranks([e0.elapsed_time(e1)])[0] / args.steps

        def ours_step(b):
            return ops[b]()[0][0]
        e2e_ms = time_e2e(ours_step, dst_dev)
        for o in ops:
            o.check()
            validate(o.out[0], "end-to-end op")
        clocks = sampler.stop() if sampler else None
        e2e_tflops = 2.0 * M * N * K / (e2e_ms * 1e-3) / 1e12
        for o in ops:
            if o is not op:
                o.close()

        # ---- same-box comparison: cuBLAS GEMM + NCCL all-gather, timed the same way ----
        base = None
        if not args.no_baseline:
            b_kn = bt_local.t()
            c_part = torch.empty((M, n_local), dtype=torch.bfloat16, device=dev)
            gathered = torch.empty((world, M, n_local), dtype=torch.bfloat16, device=dev)

            def unfused():
                torch.matmul(a_dev, b_kn, out=c_part)
                if world > 1:
                    dist.all_gather_into_tensor(gathered, c_part)
            for _ in range(args.warmup):
                unfused()
            bst = _stats(timed_steps(unfused, args.steps))
            base_ms = bst["median"]
            # end to end: the same sharded copy, NCCL all-gather of A, cuBLAS, NCCL all-gather of C, one row back
            if world == 1:
                a_in = [a_dev, torch.empty_like(a_dev)]
                base_dst = a_in
            else:
                base_dst = [torch.empty((ms_rows, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]
                a_in = [torch.empty((M, K), dtype=torch.bfloat16, device=dev) for _ in range(2)]

            def base_step(b):
                if world > 1:
                    dist.all_gather_into_tensor(a_in[b], base_dst[b])
                torch.matmul(a_in[b], b_kn, out=c_part)
                if world > 1:
                    dist.all_gather_into_tensor(gathered, c_part)
                    return gathered[:, 0, :]     # row 0 of C: one piece per rank's column block
                return c_part[0]
            base_e2e_ms = time_e2e(base_step, base_dst)
            base = {"impl": "cuBLAS + NCCL all_gather_into_tensor", "ms_per_step": round(base_ms, 4),
                    "tflops": round(2.0 * M * N * K / (base_ms * 1e-3) / 1e12, 1), "per_step_ms": bst,
                    "e2e": {"ms_per_step": round(base_e2e_ms, 4),
                            "value": round(2.0 * M * N * K / (base_e2e_ms * 1e-3) / 1e12, 2), "unit": "TFLOP/s",
                            "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": rows_host[0].numel() * 2}}

        out = {
            "metric": "fused GEMM+all-scatter TFLOPS (2MNK/time, device-timed, max over ranks)",
            "value": round(tflops, 2), "unit": "TFLOP/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": round(ms_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(tflops / base["tflops"], 3) if base else None, "dtype": "bf16", "data": "synthetic",
            "impl": "ours",
            "config": {"model": "GEMM+all-scatter A[8192,4096] x B[4096,14336], B column-sharded",
                       "global_batch": M, "seq_len": K, "parallelism": f"tp{world}",
                       "tile": f"{128 * op.cta_group}x{op.bn}x64", "push_kind": op.push_kind, "heap_mode": ctx.heap_mode,
                       "l2": "inputs larger than L2 (A 64 MB + B shard + C 235 MB rewritten every step)",
                       "timing": "one CUDA-event pair per step, max over ranks per step, ms_per_step = median",
                       "baseline_note": "vs_baseline = value / TFLOP/s of cuBLAS + NCCL all-gather measured in this "
                                        "run (same_box_baseline); the reference publishes no figure for this "
                                        "configuration"},
            "per_step_ms": dict(st, steps=[round(x, 4) for x in per_step]),
            "e2e": {"value": round(e2e_tflops, 2), "unit": "TFLOP/s", "ms_per_step": round(e2e_ms, 4),
                    "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": rows_host[0].numel() * 2,
                    "input": "whole A per step" if world == 1 else
                             "M / N rows of A per rank per step; the kernel's all-gather prologue distributes them"},
            "gpu_launches": launches,
            "clocks": clocks,
            "selfcheck": selfcheck,
            "same_box_baseline": base,
        }
        op.close()
    except Exception as exc:  # report, so that the record says why there is no number
        out = {"error": f"rank {rank}: {type(exc).__name__}: {exc}", "impl": "ours", "n_gpus": world}
        print(json.dumps(out), flush=True)
        raise
    failed = bool(out.get("selfcheck")) and any(not (isinstance(v, float) and v <= 1.0)
                                                 for v in out["selfcheck"].values())
    if rank == 0:
        print(json.dumps(out), flush=True)
    barrier()
    if world > 1:
        dist.destroy_process_group()
    return 1 if failed else 0


def run_selfcheck(ctx, G, torch, dist, dev, rank, world, barrier):
    """GEMM + all-reduce (atomic, one-shot, two-shot, push two-shot), GEMM + reduce-scatter and all-gather -> GEMM between the real
    GPUs of this run, each called three times back to back without a host barrier, against an fp32 product of the
    unsharded operands.  Returns {name: worst error / tolerance over the ranks} (<= 1 passes)."""
    mark = ctx.mark()
    res = {}

    def rnd(shape, seed, scale=1.0):
        g = torch.Generator(device=dev).manual_seed(seed)
        return (torch.randn(shape, generator=g, device=dev) * scale).to(torch.bfloat16)

    def ratio(got, ref, scale, ulps):
        tol = ulps * 2.0 ** -8 * scale + 1e-3 * ref.abs().max().item() + 1e-6
        return float(((got.float() - ref).abs() / tol).max().item())

    m, n, ks = 256 * world, 512, 384
    a_full, b_full = rnd((m, ks * world), 101), rnd((n, ks * world), 102, 0.05)
    a_l, b_l = a_full[:, rank * ks:(rank + 1) * ks], b_full[:, rank * ks:(rank + 1) * ks]
    parts = [a_full[:, r * ks:(r + 1) * ks].float() @ b_full[:, r * ks:(r + 1) * ks].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for name in ("atomic", "one_shot", "two_shot", "two_shot_push", "reduce_scatter"):
        try:
            if name == "reduce_scatter":
                op = G.gemm_reduce_scatter(ctx, [a_l], [b_l])
                rows = slice(rank * 256, (rank + 1) * 256)
            else:
                op = G.gemm_all_reduce(ctx, [a_l], [b_l], variant=name)
                rows = slice(0, m)
            barrier()
            for _ in range(3):
                o = op()[0]
            barrier()
            op.check()
            res[name] = ratio(o, ref[rows], scale[rows], 2.0 + world)
            op.close()
        except Exception as exc:
            res[name] = f"{type(exc).__name__}: {exc}"
        ctx.reset(mark)
    # all-gather -> GEMM: new rows every call, no host barrier in between
    try:
        k2, n2 = 512, 256
        bt2 = rnd((n2, k2), 110 + rank, 0.05)
        a_calls = [rnd((m, k2), 120 + c) for c in range(3)]
        op = G.all_gather_gemm(ctx, m, [bt2], ag_slices=4)
        kept = []
        barrier()
        for c in range(3):
            op.a_full[0][rank * 256:(rank + 1) * 256].copy_(a_calls[c][rank * 256:(rank + 1) * 256])
            kept.append(op()[0].clone())
        barrier()
        op.check()
        worst = 0.0
        for c in range(3):
            r = a_calls[c].float() @ bt2.float().t()
            worst = max(worst, ratio(kept[c], r, r.abs(), 2.0))
        res["all_gather_gemm"] = worst
        op.close()
    except Exception as exc:
        res["all_gather_gemm"] = f"{type(exc).__name__}: {exc}"
    ctx.reset(mark)
    # worst ratio over the ranks (a failure text on any rank wins)
    for name, v in list(res.items()):
        t = torch.tensor([v if isinstance(v, float) else float("inf")], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        if isinstance(v, float):
            res[name] = round(float(t.item()), 4) if t.item() != float("inf") else "failed on another rank"
    return res


if __name__ == "__main__":
    sys.exit(main())
