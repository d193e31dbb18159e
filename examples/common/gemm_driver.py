"""Driver shared by the fused GEMM + collective examples 07 / 08 / 09 / 11.

Role in the reference: ``examples/07_gemm_all_scatter/benchmark.py:24-299`` and its two copies (argument parsing,
operand set-up with a fixed seed, sharding, validation against ``A @ B``, timing, JSON).  Differences: time is
taken on the device around the fused launch only (plus the output clear the atomic variant needs), ranks are
aligned by a barrier before every iteration, and the figure reported is the maximum over ranks; the unfused
cuBLAS + NCCL time for the same shape is measured next to it; the roofline fraction is printed.
"""
from __future__ import annotations

import argparse

from .harness import device_barrier, iris, reduce_ranks, time_kernel_ms, torch
from iris_b200.ops import gemm as G
from iris_b200.utils import roofline
from iris_b200.utils.results import JSONWriter


def parse_args(kind: str):
    d = {"all_scatter": dict(m=8192, n=14336, k=4096), "atomic": dict(m=8192, n=4096, k=11008),
         "one_shot": dict(m=8192, n=4096, k=11008), "reduce_scatter": dict(m=16384, n=4096, k=14336)}[kind]
    ap = argparse.ArgumentParser(description=f"Fused GEMM + {kind}", formatter_class=argparse.ArgumentDefaultsHelpFormatter)
    ap.add_argument("-m", type=int, default=d["m"])
    ap.add_argument("-n", type=int, default=d["n"])
    ap.add_argument("-k", type=int, default=d["k"])
    ap.add_argument("-d", "--debug", action="store_true")
    ap.add_argument("-v", "--validate", action="store_true")
    ap.add_argument("-t", "--trace_tiles", action="store_true", help="record per-tile device timestamps to trace_rank<r>.json")
    ap.add_argument("-b", "--benchmark", action="store_true")
    ap.add_argument("--datatype", default="bf16", choices=["fp16", "fp32", "int8", "bf16"],
                    help="element type of A, B and C: bf16 / fp16 (fp32 accumulation) for every kernel; fp32 (multiplied "
                         "as tf32) and int8 (int32 accumulation, low 8 bits stored) for the all-scatter kernel")
    ap.add_argument("--output_file", default="")
    ap.add_argument("--gsize_m", type=int, default=8, help="m-tiles per raster group")
    ap.add_argument("--heap_size", type=int, default=1 << 31)
    ap.add_argument("--gemm_sms", type=int, default=0, help="CTAs of the persistent grid (0: one per SM)")
    ap.add_argument("--variant", default=None,
                    help="all-reduce only: atomic | one_shot | two_shot | two_shot_push | auto")
    ap.add_argument("--BLK_M", type=int, default=None, choices=[128, 256],
                    help="tile rows: 128 (one CTA per tile) or 256 (a CTA pair per tile); default: chosen from M")
    ap.add_argument("--BLK_N", type=int, default=None, choices=[64, 128, 256], help="tile columns (default 256)")
    ap.add_argument("--tail_split", type=int, default=0,
                    help="cut the tiles of a ragged last wave into up to this many column pieces (0: off)")
    ap.add_argument("--push_kind", default=None, choices=["tma", "tma_spread", "stores", "multimem"],
                    help="all-scatter / atomic: how tiles travel to the other ranks")
    ap.add_argument("--all_gather", action="store_true",
                    help="all-scatter only: A arrives row-sharded (M / ranks rows per rank) and the kernel's all-gather "
                         "prologue distributes it while the tiles of rows already present are computed")
    ap.add_argument("--ksplit", type=int, default=None, help="atomic / one-shot on short matrices: K pieces per tile")
    ap.add_argument("--num_experiments", type=int, default=50)
    ap.add_argument("--num_warmup", type=int, default=10)
    ap.add_argument("--no_baseline", action="store_true")
    ap.add_argument("--heap_mode", default=None, choices=["ipc", "vmm"],
                    help="vmm + IRIS_NVLS=1 in the environment binds the heap to an NVLS multicast object")
    # knobs of the reference that have no meaning on this hardware are accepted and ignored
    for flag in ("--BLK_K", "--num_stages", "--num_warps", "--waves_per_eu", "--mfmaInstrSize", "--kpack",
                 "--total_sms"):
        ap.add_argument(flag, type=int, default=None, help=argparse.SUPPRESS)
    ap.add_argument("--two_tiles", default="True", help=argparse.SUPPRESS)
    ap.add_argument("--algorithm", default=None, help=argparse.SUPPRESS)
    return vars(ap.parse_args())


def run(kind: str, seed: int):
    args = parse_args(kind)
    ctx = iris.iris(args["heap_size"], heap_mode=args["heap_mode"])
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    dbar = device_barrier(ctx)   # allocated first, in the same order on every rank
    m, n, k = args["m"], args["n"], args["k"]
    gen = torch.Generator(device=dev).manual_seed(seed)  # same seed everywhere -> identical A and B
    dtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32": torch.float32, "int8": torch.int8}[args["datatype"]]
    if dtype in (torch.float32, torch.int8) and kind != "all_scatter":
        raise SystemExit("fp32 and int8 are offered by the all-scatter kernel only (the reductions are 16-bit)")
    if dtype == torch.int8:
        A = torch.randint(-128, 128, (m, k), generator=gen, device=dev, dtype=torch.int32).to(dtype)
        Bt = torch.randint(-128, 128, (n, k), generator=gen, device=dev, dtype=torch.int32).to(dtype)
    else:
        A = (torch.randn((m, k), generator=gen, device=dev) * 0.02).to(dtype)
        Bt = (torch.randn((n, k), generator=gen, device=dev) * 0.02).to(dtype)  # B = Bt.T, K-major
    if dtype == torch.float32:
        torch.backends.cuda.matmul.allow_tf32 = True   # the library arm multiplies as tf32 too
    ctas = args["gemm_sms"] or None
    # tile shape and schedule knobs (the reference's BLK_M / BLK_N, examples/07_gemm_all_scatter/benchmark.py:53-60)
    tile_kw = dict(bn=args["BLK_N"], cta_group={None: None, 128: 1, 256: 2}[args["BLK_M"]])
    if args["tail_split"] > 1:
        tile_kw["tail_split"] = args["tail_split"]
    peaks = roofline.load_peaks()
    import torch.distributed as dist
    if kind == "all_scatter":
        if n % world:
            raise SystemExit("N must be divisible by the number of ranks")
        nl = n // world
        bt_local = Bt[rank * nl:(rank + 1) * nl].contiguous()
        if args["all_gather"]:
            if m % world:
                raise SystemExit("M must be divisible by the number of ranks")
            op = G.FusedGemm(ctx, None, [bt_local], "store", M=m, ag=True, store_all=True, c_cols=n,
                             col_off_per_rank=nl, ctas_per_rank=ctas, group_m=args["gsize_m"],
                             trace=args["trace_tiles"], push_kind=args["push_kind"], **tile_kw)
            rows = slice(rank * (m // world), (rank + 1) * (m // world))
            op.a_full[0][rows].copy_(A[rows])       # this rank's rows only; the kernel fetches the rest
        else:
            op = G.gemm_all_scatter(ctx, [A], [bt_local], ctas_per_rank=ctas, group_m=args["gsize_m"],
                                    trace=args["trace_tiles"], push_kind=args["push_kind"], **tile_kw)
        roof = roofline.all_scatter_roofline_us(m, n, k, world, peaks, args["datatype"])
        c_part = torch.empty((m, nl), dtype=dtype, device=dev)
        gathered = torch.empty((world, m, nl), dtype=dtype, device=dev)

        def unfused():
            torch.cuda.nvtx.range_push("GEMM")
            if dtype == torch.int8:   # the library's int8 GEMM returns the int32 sums; the cast keeps their low 8 bits
                c_part.copy_(torch._int_mm(A, bt_local.t()))
            else:
                torch.matmul(A, bt_local.t(), out=c_part)
            torch.cuda.nvtx.range_pop()
            if world > 1:
                torch.cuda.nvtx.range_push("Communication")
                dist.all_gather_into_tensor(gathered, c_part)
                torch.cuda.nvtx.range_pop()
        a_local, b_local = A, bt_local
        variant = "all_scatter"
    elif kind == "reduce_scatter":
        if k % world or (k // world) % 8:
            raise SystemExit("K / ranks must be a multiple of 8")
        ks = k // world
        a_local, b_local = A[:, rank * ks:(rank + 1) * ks], Bt[:, rank * ks:(rank + 1) * ks]
        tile_kw.pop("tail_split", None)
        op = G.gemm_reduce_scatter(ctx, [a_local], [b_local], ctas_per_rank=ctas, group_m=args["gsize_m"],
                                   trace=args["trace_tiles"], **tile_kw)
        roof = roofline.all_reduce_roofline_us(m, n, k, world, peaks, "reduce_scatter")
        c_part = torch.empty((m, n), dtype=dtype, device=dev)
        c_kept = torch.empty((m // world, n), dtype=dtype, device=dev)

        def unfused():
            torch.matmul(a_local, b_local.t(), out=c_part)
            if world > 1:
                dist.reduce_scatter_tensor(c_kept, c_part)
        variant = "reduce_scatter"
    else:
        variant = args["variant"] or kind
        if k % world or (k // world) % 8:
            raise SystemExit("K / ranks must be a multiple of 8")
        ks = k // world
        a_local, b_local = A[:, rank * ks:(rank + 1) * ks], Bt[:, rank * ks:(rank + 1) * ks]  # views, pitch k
        extra = {k_: v for k_, v in tile_kw.items() if v is not None}
        if args["ksplit"]:
            extra["ksplit"] = args["ksplit"]
        if args["push_kind"] and variant == "atomic":
            extra["push_kind"] = args["push_kind"]
        if variant != "atomic":
            extra.pop("tail_split", None)
        op = G.gemm_all_reduce(ctx, [a_local], [b_local], variant=variant, ctas_per_rank=ctas, group_m=args["gsize_m"],
                               trace=args["trace_tiles"], **extra)
        variant = {"store": "?", "reduce": "atomic"}.get(op.mode, "two_shot_push" if op.bcast else op.mode)
        roof = roofline.all_reduce_roofline_us(m, n, k, world, peaks,
                                               "two_shot" if variant.startswith("two_shot") else "one_shot")
        c_part = torch.empty((m, n), dtype=dtype, device=dev)

        def unfused():
            torch.matmul(a_local, b_local.t(), out=c_part)
            if world > 1:
                dist.all_reduce(c_part)
    js = JSONWriter(args["output_file"] if rank == 0 else "")
    fields = {k_: v for k_, v in args.items() if v is not None}
    fields.update(world_size=world, variant=variant, gemm_sms=op.ctas_per_rank,
                  tile=f"{128 * op.cta_group}x{op.bn}x{128 // A.element_size()}", ksplit=op.ksplit, push_kind=op.push_kind,
                  tail=[op.tail_tiles, op.tail_split])
    res = op.resources()
    if res:  # the reference's gemm_registers / gemm_spills (examples/07_gemm_all_scatter/benchmark.py:237-242)
        fields.update(gemm_registers=res["registers"], gemm_spills=res["spill_store_bytes"] + res["spill_load_bytes"])
    js.add_fields(**fields)
    js.add_environment(dev)
    G.matmul.set_debug(args["debug"])
    ctx.barrier()
    if dbar is not None:   # the ranks' streams start the validated / traced call together
        torch.cuda._sleep(1000000)
        dbar()
    out = G.matmul.apply(op)
    ctx.barrier()
    op.check()
    if args["trace_tiles"]:
        import json
        with open(f"trace_rank{rank}.json", "w") as f:
            json.dump(op.trace_records(), f)
        op.chrome_trace(f"trace_rank{rank}.chrome.json")
        ctx.log(f"per-tile trace written to trace_rank{rank}.json (records) and trace_rank{rank}.chrome.json (timeline)")
    ok = True
    if args["validate"]:
        rows = slice(0, min(m, 1024))
        got = out[rows]
        if kind == "reduce_scatter":  # this rank holds rows [rank * m / world, ...) only
            rows = slice(rank * (m // world), rank * (m // world) + min(m // world, 1024))
            got = out[:rows.stop - rows.start]
        if dtype == torch.int8:   # exact: the low 8 bits of the integer sums
            full = (A[rows].double() @ Bt.double().t()).to(torch.int64)
            ok = torch.equal(got, (((full + 128) % 256) - 128).to(torch.int8))
        elif dtype == torch.float32:   # two tf32 roundings (2^-11 each) per product
            ref = A[rows].double() @ Bt.double().t()
            tol = 2.0 ** -9 * (A[rows].double().abs() @ Bt.double().abs().t())
            ok = bool(((got.double() - ref).abs() <= tol + 1e-9).all())
        else:
            ref = A[rows].float() @ Bt.float().t()
            # bf16 rounding of the result and (all-reduce) of the partials, relative to the largest entry
            err = (got.float() - ref).abs().max().item()
            ok = err <= (2.0 + world) * 2.0 ** -8 * ref.abs().max().item()
        ctx.log(f"Validation {'successful' if ok else 'FAILED'}.")
        js.add_field("success", ok)
    if args["benchmark"]:
        def fused():  # range names as in the reference (examples/07_gemm_all_scatter/benchmark.py:179-180)
            torch.cuda.nvtx.range_push("GEMM + Communication")
            op()
            torch.cuda.nvtx.range_pop()
        ms = time_kernel_ms(ctx, fused, args["num_warmup"], args["num_experiments"], align=True)
        ms = reduce_ranks(ctx, ms, "max")
        op.check()
        flops = 2.0 * m * n * k
        tflops = flops / (ms * 1e-3) / 1e12
        frac = roof["target_us"] / (ms * 1e3)
        js.add_fields(fused_ms=ms, fused_tflops=tflops, roofline_us=roof["target_us"], roofline_bound=roof["bound"],
                      roofline_fraction=frac, peaks=peaks.source)
        line = (f"{variant} W={world} M={m} N={n} K={k}: fused {ms * 1e3:.1f} us = {tflops:.1f} TFLOPS, "
                f"roofline {roof['target_us']:.0f} us ({roof['bound']}-bound) -> {100 * frac:.0f}% of {peaks.source}")
        if not args["no_baseline"]:
            if world > 1 and not dist.is_initialized():
                raise SystemExit("baseline needs torch.distributed")
            bms = reduce_ranks(ctx, time_kernel_ms(ctx, unfused, args["num_warmup"], args["num_experiments"], align=True), "max")
            js.add_fields(baseline_ms=bms, baseline_tflops=flops / (bms * 1e-3) / 1e12, speedup=bms / ms)
            line += f" | cuBLAS+NCCL {bms * 1e3:.1f} us -> speed-up {bms / ms:.2f}x"
        if rank == 0:
            print(line, flush=True)
    if rank == 0:
        js.flush()
    op.close()
    ctx.barrier()
    ctx.close()
    if not ok:
        raise SystemExit(1)
