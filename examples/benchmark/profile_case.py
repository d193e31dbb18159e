#!/usr/bin/env python
"""Run a few launches of one fused kernel on ONE GPU, sized for a profiler capture (inputs above the L2 size,
well under a few GB).  With ``--world W > 1`` the W ranks are simulated by one launch on the GPU, so the
collective epilogue (pushes, flags, pulls) shows up in the same capture as the tensor-core tiles.

    python examples/benchmark/profile_case.py --workload one_shot --world 2
    ncu --set full --clock-control none -k regex:fused_gemm_kernel -s 1 -c 2 -o prof \\
        python examples/benchmark/profile_case.py --workload one_shot --world 2

Role in the reference: ``scripts/profile.sh`` (a rocprof-sys wrapper around one example run).
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from common.harness import iris, torch  # noqa: E402

from iris_b200.ops import gemm as G  # noqa: E402


def run_p2p(args):
    """The bandwidth kernels between two heaps on ONE GPU: the 'remote' heap is local memory, so the capture shows the
    kernels' own DRAM efficiency (256 MB buffers, larger than L2); across GPUs the same kernels are link-bound."""
    from iris_b200.ops import p2p
    ranks = iris.Iris.local_world(2, heap_size=(3 << 28) + (1 << 26))
    c = ranks[0]
    n = 1 << 26  # fp32 elements = 256 MB
    src = [r.ones(n, dtype=torch.float32) for r in ranks]
    dst = [r.zeros(n, dtype=torch.float32) for r in ranks]
    for _ in range(args.launches):
        p2p.load(c, src[0], dst[0], target=1)
        p2p.store(c, dst[0].view(torch.int32), target=1)
        p2p.all_load(c, src[0], dst[0])
        p2p.atomic_add_f32(c, dst[0], target=1, n=1 << 24)
    torch.cuda.synchronize()
    print(f"p2p kernels on one GPU: {args.launches} rounds of load / store / all_load / atomic_add")
    ranks[0].close()


def run_mp(args):
    """The message-passing kernel with producer and consumer blocks in ONE cooperative launch on one GPU (64 chunks of
    1 MB): the copy, the per-slice publish and the consumer's pass, without a link in between."""
    from iris_b200.ops import p2p
    ranks = iris.Iris.local_world(2, heap_size=1 << 29)
    # the same allocations, in the same order, on both simulated ranks (symmetric offsets)
    mps = [p2p.MessagePassing(r, nchunks=64, chunk_bytes=1 << 20, producer=0, consumer=1, timeout_ms=2000)
           for r in ranks]
    mps[0].src.copy_(torch.arange(mps[0].src.numel(), device="cuda", dtype=torch.float32) % 1000)
    for _ in range(args.launches):
        for m in mps:
            m.epoch += 1
        mps[0].run(roles=3, advance=False)
    torch.cuda.synchronize()
    ranks[1].check_status()
    assert torch.equal(mps[1].out, 2 * mps[0].src)
    print(f"message passing on one GPU: {args.launches} hand-offs of 64 x 1 MB, {mps[0].parts} slices per chunk")
    ranks[0].close()


def run_elementwise(args):
    """RMSNorm, SwiGLU and residual add on 16384 x 4096 (x 11008) bf16 activations: memory-bound kernels."""
    from iris_b200.ops import elementwise as E
    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn((16384, 4096), generator=g, device="cuda").to(torch.bfloat16)
    y = torch.randn((16384, 4096), generator=g, device="cuda").to(torch.bfloat16)
    w = torch.ones(4096, device="cuda", dtype=torch.bfloat16)
    out = torch.empty_like(x)
    gu = torch.randn((16384, 2 * 1376), generator=g, device="cuda").to(torch.bfloat16)
    h = torch.empty((16384, 1376), device="cuda", dtype=torch.bfloat16)
    for _ in range(args.launches):
        E.rmsnorm(x, w, out, 1e-6)
        E.swiglu(gu, h)
        E.residual_add(x, y)
        E.add_rmsnorm(x, y, w, out, 1e-6)
    torch.cuda.synchronize()
    print(f"elementwise kernels: {args.launches} rounds of rmsnorm / swiglu / residual_add / add_rmsnorm")


def run_attention(args):
    """The tcgen05 attention kernel on batch 8 x seq 2048 x 4 heads of 128 (48 MB of qkv), causal."""
    from iris_b200.ops.attention import attention_fwd
    batch, seq, heads = 8, 2048, 4
    g = torch.Generator(device="cuda").manual_seed(1)
    dt = torch.float16 if args.dtype == "fp16" else torch.bfloat16
    qkv = torch.randn((batch * seq, 3 * heads * 128), generator=g, device="cuda").to(dt)
    out = torch.empty((batch * seq, heads * 128), dtype=dt, device="cuda")
    for _ in range(args.launches):
        attention_fwd(qkv, out, batch, seq, heads)
    torch.cuda.synchronize()
    print(f"attention: {args.launches} launches, batch {batch} x seq {seq} x {heads} heads, {args.dtype}")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="gemm", choices=["gemm", "all_scatter", "atomic", "one_shot", "two_shot", "reduce_scatter", "ag", "p2p",
                             "mp", "elementwise", "attention"])
    ap.add_argument("--world", type=int, default=1)
    ap.add_argument("-m", type=int, default=8192)
    ap.add_argument("-n", type=int, default=3584)
    ap.add_argument("-k", type=int, default=4096)
    ap.add_argument("--launches", type=int, default=3)
    ap.add_argument("--cta_group", type=int, default=0)
    ap.add_argument("--bn", type=int, default=0, help="tile width: 64, 128 or 256 (0: the default, 256)")
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "fp16", "fp32", "int8"],
                    help="fp32 (multiplied as tf32) and int8: workloads gemm, all_scatter and ag only")
    args = ap.parse_args()
    W = args.world
    if args.workload == "p2p":
        return run_p2p(args)
    if args.workload == "mp":
        return run_mp(args)
    if args.workload == "elementwise":
        return run_elementwise(args)
    if args.workload == "attention":
        return run_attention(args)
    ranks = iris.Iris.local_world(W, heap_size=(1 << 30) // max(1, W // 2))
    g = torch.Generator(device="cuda").manual_seed(0)

    dt = {"fp16": torch.float16, "fp32": torch.float32, "int8": torch.int8}.get(args.dtype, torch.bfloat16)

    def rand(r, c):
        if dt == torch.int8:
            return torch.randint(-128, 128, (r, c), generator=g, device="cuda", dtype=torch.int32).to(dt)
        return (torch.randn((r, c), generator=g, device="cuda") * 0.02).to(dt)
    cg = args.cta_group or None
    bn = args.bn or None
    m, n, k = args.m, args.n, args.k
    if args.workload in ("gemm", "all_scatter"):
        a = rand(m, k)
        bts = [rand(n // W, k) for _ in range(W)]
        op = G.gemm_all_scatter(ranks, [a] * W, bts, cta_group=cg, bn=bn)
    elif args.workload == "ag":
        bts = [rand(n // W, k) for _ in range(W)]
        op = G.all_gather_gemm(ranks, m, bts, cta_group=cg, bn=bn)
        for r in range(W):
            op.a_full[r][r * (m // W):(r + 1) * (m // W)].copy_(rand(m // W, k))
    else:
        ks = k // W
        a_full, b_full = rand(m, k), rand(n, k)
        a_sh = [a_full[:, r * ks:(r + 1) * ks] for r in range(W)]
        b_sh = [b_full[:, r * ks:(r + 1) * ks] for r in range(W)]
        if args.workload == "reduce_scatter":
            op = G.gemm_reduce_scatter(ranks, a_sh, b_sh, cta_group=cg, bn=bn)
        else:
            op = G.gemm_all_reduce(ranks, a_sh, b_sh, variant=args.workload, cta_group=cg, bn=bn)
    for _ in range(args.launches):
        op()
    op.check()
    print(f"{args.workload} W={W} {m}x{n}x{k} {args.dtype}: {args.launches} launches, tile {128 * op.cta_group}x{op.bn}, "
          f"ctas/rank={op.ctas_per_rank}")
    op.close()
    ranks[0].close()


if __name__ == "__main__":
    main()
