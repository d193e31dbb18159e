"""Worker run as one process per GPU with heap_mode="vmm": file-descriptor exchange, contiguous mapping of all
heaps, remote access through it and — when IRIS_NVLS=1 and the machine offers it — multicast stores and
switch-side all-reduce, each checked exactly or against PyTorch."""
import os
import sys

import torch

import iris_b200 as iris
from iris_b200.ops import nvls


def main():
    ctx = iris.iris(256 << 20, heap_mode="vmm")
    rank, world = ctx.get_rank(), ctx.get_num_ranks()
    dev = ctx.get_device()
    hb = [int(x) for x in ctx.get_heap_bases().cpu().tolist()]
    stride = hb[1] - hb[0]
    assert all(hb[r] == hb[0] + r * stride for r in range(world)), "heaps are not contiguous in the address space"
    buf = ctx.zeros(4096, dtype=torch.float32)
    ctx.barrier()
    iris.store(ctx, buf, float(rank + 1), target=(rank + 1) % world, block=256)
    ctx.barrier()
    assert torch.equal(buf, torch.full_like(buf, float((rank - 1) % world + 1)))
    acc = ctx.zeros(64, dtype=torch.int32)
    ctx.barrier()
    iris.atomic_add(ctx, acc, 1, sem="relaxed", scope="sys", block=64)
    ctx.barrier()
    assert torch.equal(acc, torch.full_like(acc, world))
    msg = f"rank {rank}: VMM OK"
    if os.environ.get("IRIS_NVLS") == "1":
        if not nvls.available(ctx):
            msg += " (NVLS not available on this machine)"
        else:
            words = ctx.zeros(1 << 18, dtype=torch.int32)
            ctx.barrier()
            if rank == 0:
                nvls.all_store(ctx, words)
            ctx.barrier()
            assert torch.equal(words, torch.arange(words.numel(), dtype=torch.int32, device=dev)), "multimem.st"
            ar = nvls.AllReduce(ctx)
            x = ctx.zeros(1 << 20, dtype=torch.bfloat16)
            for it in range(3):
                g = torch.Generator(device=dev).manual_seed(100 + it)
                parts = [torch.randn(x.numel(), generator=g, device=dev).to(torch.bfloat16) for _ in range(world)]
                x.copy_(parts[rank])
                ctx.barrier()
                ar(x)
                ctx.barrier()
                ctx.check_status()
                ref = sum(p.float() for p in parts)
                assert (x.float() - ref).abs().max().item() <= 2 ** -7 * ref.abs().max().item(), "multimem.ld_reduce"
            # fused GEMM + two-shot all-reduce with the switch doing the summing and the broadcast
            from iris_b200.ops import gemm as G
            k_full = 1024 * world
            g = torch.Generator(device=dev).manual_seed(5)
            a_full = torch.randn((512, k_full), generator=g, device=dev).to(torch.bfloat16)
            b_full = (torch.randn((768, k_full), generator=g, device=dev) * 0.05).to(torch.bfloat16)
            ks = k_full // world
            op = G.gemm_all_reduce(ctx, [a_full[:, rank * ks:(rank + 1) * ks]], [b_full[:, rank * ks:(rank + 1) * ks]],
                                   variant="two_shot")
            assert op.nvls, "two-shot did not pick the NVLS reducer"
            for _ in range(3):
                ctx.barrier()
                o = op()[0]
            ctx.barrier()
            op.check()
            parts = [a_full[:, r * ks:(r + 1) * ks].float() @ b_full[:, r * ks:(r + 1) * ks].float().t()
                     for r in range(world)]
            ref, scale = sum(parts), sum(p.abs() for p in parts)
            tol = (2 + world) * 2.0 ** -8 * scale + 1e-3 * ref.abs().max().item()
            assert bool(((o.float() - ref).abs() <= tol).all()), "NVLS two-shot mismatch"
            op.close()
            # push two-shot: partial tiles pushed to the keeper of their rows, summed there, result rows delivered to
            # every rank with multimem stores
            if 512 % (world * 128) == 0:
                tp = G.gemm_all_reduce(ctx, [a_full[:, rank * ks:(rank + 1) * ks]],
                                       [b_full[:, rank * ks:(rank + 1) * ks]], variant="two_shot_push")
                assert tp.nvls and tp.bcast
                for _ in range(3):
                    o = tp()[0]
                ctx.barrier()
                tp.check()
                assert bool(((o.float() - ref).abs() <= tol).all()), "NVLS push two-shot mismatch"
                tp.close()
            # fused GEMM + all-scatter whose tiles leave as multimem stores: one store per 16 bytes, the switch
            # delivers it to every rank's C (this rank's own copy included)
            n_local = 320
            a = torch.randn((1000, 512), generator=g, device=dev).to(torch.bfloat16)
            bts = [(torch.randn((n_local, 512), generator=g, device=dev) * 0.05).to(torch.bfloat16)
                   for _ in range(world)]
            sc = G.gemm_all_scatter(ctx, [a], [bts[rank]], push_kind="multimem")
            assert sc.push_kind == "multimem"
            for _ in range(3):
                c = sc()[0]
            ctx.barrier()
            sc.check()
            ref = torch.cat([a.float() @ b.float().t() for b in bts], dim=1)
            assert bool(((c.float() - ref).abs() <= 2.0 ** -7 * ref.abs() + 1e-3 * ref.abs().max().item()).all()), \
                "multimem all-scatter mismatch"
            sc.close()
            # atomic all-reduce of a short matrix: every 64-column tile is added into all ranks' outputs by the
            # switch (one multimem.red per 16 bytes)
            ar = G.gemm_all_reduce(ctx, [a_full[:128, rank * ks:(rank + 1) * ks]],
                                   [b_full[:, rank * ks:(rank + 1) * ks]], variant="atomic", bn=64,
                                   push_kind="multimem")
            assert ar.push_kind == "multimem" and ar.bn == 64
            for _ in range(3):
                o = ar()[0]
            ctx.barrier()
            ar.check()
            parts = [a_full[:128, r * ks:(r + 1) * ks].float() @ b_full[:, r * ks:(r + 1) * ks].float().t()
                     for r in range(world)]
            ref, scale = sum(parts), sum(p.abs() for p in parts)
            tol = (2 + 2 * world) * 2.0 ** -8 * scale + 1e-3 * ref.abs().max().item()
            assert bool(((o.float() - ref).abs() <= tol).all()), "multimem atomic all-reduce mismatch"
            ar.close()
            msg += " + NVLS OK"
    ctx.barrier()
    ctx.close()
    print(msg, flush=True)


if __name__ == "__main__":
    main()
    sys.exit(0)
