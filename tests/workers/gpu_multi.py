"""Worker run as one process per GPU (2, 4 or 8 ranks): the real inter-GPU paths — CUDA IPC mapping, remote
loads / stores / atomics over NVLink, message passing with the producer and the consumer on different GPUs,
and every fused GEMM + collective variant, each checked against PyTorch."""
import sys

import torch

import iris_b200 as iris
from iris_b200.ops import gemm as G, p2p


def rand(shape, seed, scale=1.0, dev="cuda"):
    g = torch.Generator(device=dev).manual_seed(seed)
    return (torch.randn(shape, generator=g, device=dev) * scale).to(torch.bfloat16)


def close(got, ref, scale=None, ulps=2.0):
    ref = ref.float()
    scale = ref.abs() if scale is None else scale
    tol = ulps * (2.0 ** -8) * scale + 1e-3 * ref.abs().max().item() + 1e-6
    err = (got.float() - ref).abs()
    assert not bool((err > tol).any()), f"max err {err.max().item():.4g}"


def main():
    ctx = iris.iris(512 << 20)
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    assert world >= 2 and dev.type == "cuda"
    hb = ctx.get_heap_bases()
    assert hb.numel() == world and int(hb[rank].item()) == ctx.heap_base()

    # ---- unit semantics: every rank applies the primitive to every rank (tests/unittests of the reference) ----
    for dtype in (torch.int8, torch.float16, torch.bfloat16, torch.float32):
        data, res = ctx.ones(32, dtype=dtype), ctx.zeros(32, dtype=dtype)
        dst = ctx.zeros(32, dtype=dtype)
        ctx.barrier()
        iris.load(ctx, data, res, block=32)
        iris.store(ctx, dst, 1, block=32)
        ctx.barrier()
        assert torch.equal(res, torch.full_like(res, world)), ("load", dtype)
        assert torch.equal(dst, torch.ones_like(dst)), ("store", dtype)
    for dtype in (torch.int32, torch.int64, torch.float16, torch.bfloat16, torch.float32):
        for sem in ("relaxed", "acquire", "release", "acq_rel"):
            acc = ctx.zeros(16, dtype=dtype)
            ctx.barrier()
            iris.atomic_add(ctx, acc, 1, sem=sem, scope="sys", block=16)
            ctx.barrier()
            assert torch.equal(acc, torch.full_like(acc, world)), ("atomic_add", dtype, sem)
    f = ctx.zeros(1, dtype=torch.int32)
    x = ctx.zeros(1, dtype=torch.int64)
    ctx.barrier()
    iris.atomic_cas(ctx, f, 0, world, sem="acq_rel", scope="sys", block=1)
    iris.atomic_xchg(ctx, x, world, sem="acq_rel", scope="sys", block=1)
    ctx.barrier()
    assert int(f[0]) == world and int(x[0]) == world

    # ---- rank 0 stores into rank 1 (the README example of the reference, README.md:31-70) ----
    buf = ctx.zeros(4096, dtype=torch.float32)
    ctx.barrier()
    if rank == 0:
        iris.store(ctx, buf, 1.0, target=1, block=1024)
    ctx.barrier()
    assert float(buf.sum()) == (4096.0 if rank == 1 else 0.0)

    # ---- bandwidth kernels: values ----
    n = 1 << 20
    src = ctx.full((n,), rank + 1, dtype=torch.float32)
    out = ctx.zeros(n, dtype=torch.float32)
    words = ctx.zeros(n, dtype=torch.int32)
    ctx.barrier()
    p2p.load(ctx, src, out, target=(rank + 1) % world)
    ctx.barrier()
    assert torch.equal(out, torch.full_like(out, (rank + 1) % world + 1))
    p2p.all_load(ctx, src, out)
    ctx.barrier()
    assert torch.equal(out, torch.full_like(out, sum(range(1, world + 1))))
    if rank == 0:
        p2p.all_store(ctx, words)
    ctx.barrier()
    expect = torch.arange(n, dtype=torch.int32, device=dev)
    assert torch.equal(words, expect) if rank != 0 else int(words.abs().sum()) == 0

    # ---- message passing across GPUs: 1 MB chunks, flag in the consumer's memory, release / acquire ----
    mp = p2p.MessagePassing(ctx, nchunks=8, chunk_bytes=1 << 20, producer=0, consumer=1, timeout_ms=5000)
    for epoch in (1, 2):
        if rank == 0:
            mp.src.copy_(torch.arange(mp.src.numel(), device=dev, dtype=torch.float32) % 1000 + epoch)
        ctx.barrier()
        mp.run(use_put=(epoch == 1))
        ctx.barrier()
        ctx.check_status()
        if rank == 1:
            want = 2 * (torch.arange(mp.src.numel(), device=dev, dtype=torch.float32) % 1000 + epoch)
            assert torch.equal(mp.out, want), f"message passing epoch {epoch}"

    # ---- fused GEMM + collectives ----
    m, n_local, k = 1024, 512, 1024
    a = rand((m, k), 5, dev=dev)
    bts = [rand((n_local, k), 10 + r, 0.05, dev=dev) for r in range(world)]
    op = G.gemm_all_scatter(ctx, [a], [bts[rank]])
    for _ in range(3):
        ctx.barrier()
        c = op()[0]
    ctx.barrier()
    op.check()
    close(c, torch.cat([a.float() @ b.float().t() for b in bts], dim=1))
    op.close()

    k_full = 2752 // world * world
    ks = k_full // world
    a_full, b_full = rand((384, k_full), 6, dev=dev), rand((768, k_full), 7, 0.05, dev=dev)
    parts = [a_full[:, r * ks:(r + 1) * ks].float() @ b_full[:, r * ks:(r + 1) * ks].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for variant in ("atomic", "one_shot", "two_shot"):
        ar = G.gemm_all_reduce(ctx, [a_full[:, rank * ks:(rank + 1) * ks]], [b_full[:, rank * ks:(rank + 1) * ks]],
                               variant=variant)
        for _ in range(3):
            ctx.barrier()
            o = ar()[0]
        ctx.barrier()
        ar.check()
        close(o, ref, scale=scale, ulps=2.0 + world)
        ar.close()

    # GEMM + reduce-scatter: every rank keeps its own rows of the sum, back-to-back calls without host barriers
    m_rs = 512 * world
    a_rs = rand((m_rs, k_full), 36, dev=dev)
    parts = [a_rs[:, r * ks:(r + 1) * ks].float() @ b_full[:, r * ks:(r + 1) * ks].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    rs = G.gemm_reduce_scatter(ctx, [a_rs[:, rank * ks:(rank + 1) * ks]], [b_full[:, rank * ks:(rank + 1) * ks]])
    ctx.barrier()
    for _ in range(4):
        o = rs()[0]
    ctx.barrier()
    rs.check()
    rows = slice(rank * 512, (rank + 1) * 512)
    close(o, ref[rows], scale=scale[rows], ulps=2.0 + world)
    rs.close()
    # the same partial pushes, but the keeper writes the summed rows to every rank: all-reduce made of pushes only
    tp = G.gemm_all_reduce(ctx, [a_rs[:, rank * ks:(rank + 1) * ks]], [b_full[:, rank * ks:(rank + 1) * ks]],
                           variant="two_shot_push")
    for _ in range(4):
        o = tp()[0]
    ctx.barrier()
    tp.check()
    close(o, ref, scale=scale, ulps=2.0 + world)
    tp.close()

    m2 = 256 * world
    ms = m2 // world
    a2 = rand((m2, 512), 8, dev=dev)
    ag = G.all_gather_gemm(ctx, m2, [bts[rank][:, :512]], ag_slices=4)
    for call in range(2):
        ag.a_full[0].zero_()
        ag.a_full[0][rank * ms:(rank + 1) * ms].copy_(a2[rank * ms:(rank + 1) * ms])
        ctx.barrier()
        o = ag()[0]
        ctx.barrier()
        ag.check()
        assert torch.equal(ag.a_full[0], a2), "gathered A differs"
        close(o, a2.float() @ bts[rank][:, :512].float().t())
    # four calls back to back with new rows each time and no host barrier in between: a rank may be a whole call
    # ahead of a peer; its pushes must wait until that peer has entered the same call
    a_calls = [rand((m2, 512), 80 + c, dev=dev) for c in range(4)]
    kept = []
    ctx.barrier()
    for c in range(4):
        ag.a_full[0][rank * ms:(rank + 1) * ms].copy_(a_calls[c][rank * ms:(rank + 1) * ms])
        kept.append(ag()[0].clone())
    ctx.barrier()
    ag.check()
    for c in range(4):
        close(kept[c], a_calls[c].float() @ bts[rank][:, :512].float().t())
    ag.close()
    # every way an all-scatter tile can travel between real GPUs, fp16 and a narrow tile among them
    for pk, dt, bn in (("tma_spread", torch.bfloat16, 256), ("stores", torch.float16, 128), ("stores", torch.bfloat16, 64)):
        sc = G.gemm_all_scatter(ctx, [a.to(dt)], [bts[rank].to(dt)], push_kind=pk, bn=bn)
        for _ in range(3):
            c = sc()[0]
        ctx.barrier()
        sc.check()
        close(c, torch.cat([a.to(dt).float() @ b.to(dt).float().t() for b in bts], dim=1))
        sc.close()
    # CUDA graph over real GPUs: all-scatter, two-shot all-reduce and the device barrier recorded once and replayed
    # with new operands (nothing in a launch changes from call to call: the call numbers are kept in device memory)
    from iris_b200.ops.p2p import DeviceBarrier
    ks2 = 1024 // world
    ag_in = a.clone()
    sc = G.gemm_all_scatter(ctx, [ag_in], [bts[rank]])
    ar = G.gemm_all_reduce(ctx, [ag_in[:, rank * ks2:(rank + 1) * ks2]], [bts[0][:, rank * ks2:(rank + 1) * ks2]],
                           variant="two_shot")
    db = DeviceBarrier(ctx)
    sc(), ar(), db()            # ordinary calls first
    torch.cuda.synchronize()
    ctx.barrier()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        db()
        sc()
        ar()
    for i in range(3):
        ag_in.copy_(rand(tuple(a.shape), 300 + i, dev=dev))
        ctx.barrier()
        graph.replay()
        torch.cuda.synchronize()
        ctx.barrier()
        sc.check(), ar.check()
        close(sc.out[0], torch.cat([ag_in.float() @ b.float().t() for b in bts], dim=1))
        parts = [ag_in[:, r * ks2:(r + 1) * ks2].float() @ bts[0][:, r * ks2:(r + 1) * ks2].float().t()
                 for r in range(world)]
        close(ar.out[0], sum(parts), scale=sum(p.abs() for p in parts), ulps=2.0 + world)
    sc(), ar(), db()            # and after the replays
    torch.cuda.synchronize()
    ctx.barrier()
    sc.check(), ar.check()
    sc.close(), ar.close()
    ctx.barrier()
    ctx.close()
    print(f"rank {rank}: OK", flush=True)


if __name__ == "__main__":
    main()
    sys.exit(0)
