#!/usr/bin/env python
"""Tensor-parallel Llama-style decoder stack: hidden 4096, 32 heads x 128, SwiGLU 11008, RMSNorm eps 1e-6, bf16
weights N(0, 0.02) from seed 4, activations N(0, 1) of batch 8 x seq 2048, 4 layers, forward only.
Column-parallel projections run as fused all-gather->GEMM, row-parallel ones as fused GEMM->all-reduce
(``iris_b200/models/tp_block.py``); the same network with cuBLAS + NCCL is timed next to it.  No counterpart in the
reference, whose fused kernels are the ingredients.

    python -m iris_b200.launch -np 8 examples/10_tp_block/tp_block.py -v -b
"""
import argparse
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import device_barrier, iris, reduce_ranks, time_kernel_ms, torch  # noqa: E402

from iris_b200.models.tp_block import TPConfig, TPDecoder, TPDecoderBaseline, reference_forward  # noqa: E402


def main():
    ap = argparse.ArgumentParser(formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("--hidden", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--head_dim", type=int, default=128)
    ap.add_argument("--intermediate", type=int, default=11008)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--attention", default="iris", choices=["iris", "sdpa"],
                    help="attention core of the fused stack: this repository's tcgen05 kernel or the library call")
    ap.add_argument("--variant", default="two_shot",
                    choices=["two_shot", "two_shot_push", "one_shot", "atomic", "auto", "reduce_scatter"],
                    help="row-parallel projections: an all-reduce variant, or reduce_scatter (every rank receives only its "
                         "own token rows; the baseline then uses NCCL reduce_scatter_tensor)")
    ap.add_argument("-v", "--validate", action="store_true", help="compare with the unsharded fp32 oracle (1 layer subset)")
    ap.add_argument("-b", "--benchmark", action="store_true")
    ap.add_argument("--num_experiments", type=int, default=10)
    ap.add_argument("--num_warmup", type=int, default=3)
    ap.add_argument("--heap_size", type=int, default=12 << 30)
    ap.add_argument("--output_file", default="")
    ap.add_argument("--cuda_graph", action="store_true",
                    help="benchmark: also time the fused forward pass replayed from a CUDA graph")
    ap.add_argument("--breakdown", action="store_true", help="per-phase device times (max over ranks) of one forward")
    ap.add_argument("--heap_mode", default=None, choices=["ipc", "vmm"],
                    help="vmm + IRIS_NVLS=1 in the environment binds the heap to an NVLS multicast object")
    args = ap.parse_args()
    cfg = TPConfig(hidden=args.hidden, n_heads=args.heads, head_dim=args.head_dim, intermediate=args.intermediate,
                   n_layers=args.layers, batch=args.batch, seq=args.seq)
    ctx = iris.iris(args.heap_size, heap_mode=args.heap_mode)
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    device_barrier(ctx)
    model = TPDecoder(ctx, cfg, variant=args.variant, attention=args.attention)
    base = TPDecoderBaseline(cfg, rank, world, dev, scatter=args.variant == "reduce_scatter")
    g = torch.Generator(device=dev).manual_seed(cfg.seed)
    x = torch.randn((cfg.tokens, cfg.hidden), generator=g, device=dev).to(torch.bfloat16)
    ts = cfg.tokens // world
    mine = x[rank * ts:(rank + 1) * ts]
    res = {"world": world, "variant": args.variant, "config": cfg.__dict__, "nvls": bool(ctx.mc_base),
           "attention": "iris" if model.own_attention else "sdpa"}
    ok = True
    if args.validate:
        a, b = mine.clone(), mine.clone()
        ctx.barrier()
        model.forward([a])
        model.check()
        base.forward(b)
        torch.cuda.synchronize()
        d_fb = (a.float() - b.float()).abs()
        res["fused_vs_baseline_max"], res["fused_vs_baseline_mean"] = d_fb.max().item(), d_fb.mean().item()
        ok = d_fb.mean().item() < 0.1  # library all-reduce rounds bf16 partial sums hop by hop
        if cfg.tokens * cfg.hidden <= 1 << 24:  # the oracle needs the full fp32 network on one GPU
            ref = reference_forward(x, cfg)[rank * ts:(rank + 1) * ts]
            err, berr = (a.float() - ref).abs(), (b.float() - ref).abs()
            res["fused_vs_oracle_max"], res["fused_vs_oracle_mean"] = err.max().item(), err.mean().item()
            res["baseline_vs_oracle_max"], res["baseline_vs_oracle_mean"] = berr.max().item(), berr.mean().item()
            ok = err.mean().item() < 3e-2  # the oracle decides; NCCL sums bf16 partials in another order
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}: {json.dumps({k: v for k, v in res.items() if 'vs' in k})}")
    if args.benchmark:
        a, b = mine.clone(), mine.clone()
        f_ms = reduce_ranks(ctx, time_kernel_ms(ctx, lambda: model.forward([a]), args.num_warmup,
                                                args.num_experiments, align=True), "max")
        model.check()
        b_ms = reduce_ranks(ctx, time_kernel_ms(ctx, lambda: base.forward(b), args.num_warmup,
                                                args.num_experiments, align=True), "max")
        res.update(fused_us=f_ms * 1e3, baseline_us=b_ms * 1e3, speedup=b_ms / f_ms)
        if args.cuda_graph:
            graph = model.capture([a])
            ctx.barrier()
            g_ms = reduce_ranks(ctx, time_kernel_ms(ctx, graph.replay, args.num_warmup, args.num_experiments,
                                                    align=True), "max")
            model.check()
            res.update(fused_graph_us=g_ms * 1e3, speedup_graph=b_ms / g_ms)
            if rank == 0:
                print(f"  fused, replayed from a CUDA graph: {g_ms * 1e3:.0f} us | x{b_ms / g_ms:.2f}", flush=True)
        if rank == 0:
            print(f"TP decoder x{cfg.n_layers} layers, W={world}, {cfg.tokens} tokens: fused {f_ms * 1e3:.0f} us | "
                  f"cuBLAS+NCCL {b_ms * 1e3:.0f} us | x{b_ms / f_ms:.2f}", flush=True)
    if args.breakdown:
        def phase_times(run):
            marks = []

            def tick(name):
                e = torch.cuda.Event(enable_timing=True)
                e.record()
                marks.append((name, e))
            for _ in range(2):
                marks.clear()
                ctx.barrier()
                run(tick)
            torch.cuda.synchronize()
            acc = {}
            for (n0, e0), (_, e1) in zip(marks[:-1], marks[1:]):
                acc[n0] = acc.get(n0, 0.0) + e0.elapsed_time(e1) * 1e3
            return {k_: reduce_ranks(ctx, v, "max") for k_, v in sorted(acc.items())}
        a, b = mine.clone(), mine.clone()
        f_ph = phase_times(lambda tick: model.forward([a], timers=tick))
        b_ph = phase_times(lambda tick: base.forward(b, timers=tick))
        res["breakdown_us"] = {"fused": f_ph, "baseline": b_ph}
        if rank == 0:
            print("phase (us, summed over layers)      fused    cuBLAS+NCCL")
            for k_ in f_ph:
                print(f"  {k_:<28} {f_ph[k_]:10.0f} {b_ph.get(k_, 0.0):10.0f}", flush=True)
    if rank == 0 and args.output_file:
        os.makedirs(os.path.dirname(args.output_file) or ".", exist_ok=True)
        with open(args.output_file, "w") as f:
            json.dump(res, f, indent=2, default=str)
    model.close()
    ctx.barrier()
    ctx.close()
    if not ok:
        raise SystemExit(1)


if __name__ == "__main__":
    main()
