"""tcgen05 GEMM and the fused GEMM + collective kernels against a plain PyTorch fp32 reference.

Multi-rank cases run as ONE cooperative launch over ranks simulated on a single GPU
(``Iris.local_world``): the per-tile flags, entry flags, pushes and pulls go through the same code as between
GPUs, only the transport is local.  Acceptance mirrors the reference's ``validate_gemm``
(``examples/common/validation.py:7-23``) but with a tolerance that fits bf16 outputs instead of ``atol=1..2``.
"""
import pytest
import torch

import iris_b200 as iris
from iris_b200.ops import gemm as G

pytestmark = pytest.mark.gpu

if not torch.cuda.is_available():
    pytest.skip("needs a CUDA device", allow_module_level=True)


def _rand(shape, seed, scale=1.0, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(shape, generator=g, device="cuda", dtype=torch.float32) * scale).to(dtype)


def _assert_close(got, ref_fp32, scale=None, ulps=2.0):
    """Element-wise bound: `ulps` bf16 roundings (2^-8 relative each) of `scale`, the magnitude the rounding acts
    on: |ref| for a plain GEMM, the sum of the partials' magnitudes when bf16 partials are added up."""
    ref = ref_fp32.float()
    scale = ref.abs() if scale is None else scale
    tol = ulps * (2.0 ** -8) * scale + 1e-3 * ref.abs().max().item() + 1e-6
    err = (got.float() - ref).abs()
    bad = err > tol
    assert not bool(bad.any()), f"{int(bad.sum())} mismatches, max err {err.max().item():.4g}"


@pytest.mark.parametrize("m,n,k", [(128, 256, 64), (256, 512, 256), (384, 768, 192), (1000, 520, 1376),
                                   (2048, 1792, 4096), (1, 4096, 1376)])
@pytest.mark.parametrize("cta_group", [1, 2])
def test_plain_gemm(m, n, k, cta_group):
    a, bt = _rand((m, k), 1), _rand((n, k), 2, 0.05)
    out = G.gemm(a, bt, cta_group=cta_group)
    torch.cuda.synchronize()
    _assert_close(out, a.float() @ bt.float().t())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("m,n,k,cta_group", [(384, 832, 192, 1), (1000, 520, 1376, 2), (100, 1024, 512, 1)])
def test_gemm_tile_widths_and_element_types(m, n, k, cta_group, bn, dtype):
    """The six tile shapes (128 or 256 rows x 64 / 128 / 256 columns) in both 16-bit element types, ragged edges."""
    a, bt = _rand((m, k), 1, dtype=dtype), _rand((n, k), 2, 0.05, dtype=dtype)
    out = G.gemm(a, bt, cta_group=cta_group, bn=bn)
    torch.cuda.synchronize()
    assert out.dtype == dtype
    _assert_close(out, a.float() @ bt.float().t())


def _int8_rand(shape, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-128, 128, shape, generator=g, device="cuda", dtype=torch.int32).to(torch.int8)


def _int8_ref(a, bt):
    """The low 8 bits of the exact integer product (int8 operands, sums far below 2^53: exact in float64)."""
    full = (a.double() @ bt.double().t()).to(torch.int64)
    return (((full + 128) % 256) - 128).to(torch.int8)


@pytest.mark.parametrize("bn", [64, 128, 256])
@pytest.mark.parametrize("m,n,k,cta_group", [(384, 832, 192, 1), (1000, 520, 1376, 2), (100, 1024, 516, 1),
                                             (2048, 1792, 2048, 2)])
def test_gemm_fp32_as_tf32(m, n, k, cta_group, bn):
    """float32 matrices multiplied on the tensor cores as tf32 (10-bit mantissa, fp32 accumulation), fp32 result:
    32-element K slices and 32-column epilogue sub-tiles.  Bound: two tf32 roundings per product (2^-10 relative)."""
    a, bt = _rand((m, k), 1, dtype=torch.float32), _rand((n, k), 2, 0.05, dtype=torch.float32)
    out = G.gemm(a, bt, cta_group=cta_group, bn=bn)
    torch.cuda.synchronize()
    assert out.dtype == torch.float32
    ref = a.double() @ bt.double().t()
    scale = a.double().abs() @ bt.double().abs().t()      # what the operand roundings act on
    err = (out.double() - ref).abs()
    bad = err > 2.0 ** -9 * scale + 1e-6
    assert not bool(bad.any()), f"{int(bad.sum())} mismatches, max err {err.max().item():.4g}"
    # and it is a tensor-core product, not an fp32 one: the error is visible at fp32 resolution for long K
    if k >= 1024:
        assert err.max().item() > 0


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("m,n,k,cta_group", [(384, 896, 192, 1), (1000, 528, 1376, 2), (100, 1024, 512, 1),
                                             (2048, 1792, 4096, 2)])
def test_gemm_int8(m, n, k, cta_group, bn):
    """int8 matrices, 32-bit integer accumulation, int8 result = the low 8 bits of the sum: exact."""
    a, bt = _int8_rand((m, k), 1), _int8_rand((n, k), 2)
    out = G.gemm(a, bt, cta_group=cta_group, bn=bn)
    torch.cuda.synchronize()
    assert out.dtype == torch.int8
    assert torch.equal(out, _int8_ref(a, bt))


@pytest.mark.parametrize("push_kind", ["tma", "tma_spread", "stores"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.int8])
def test_all_scatter_and_all_gather_fp32_int8(dtype, push_kind):
    """GEMM + all-scatter and all-gather + GEMM with 32- and 8-bit elements (two ranks in one cooperative launch)."""
    world, m, n_local, k = 2, 1024, 640, 512
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    if dtype == torch.int8:
        a = _int8_rand((m, k), 5)
        bts = [_int8_rand((n_local, k), 10 + r) for r in range(world)]
        refs = [_int8_ref(a, b) for b in bts]
        same = [lambda got, want=want: torch.equal(got, want) for want in refs]
    else:
        a = _rand((m, k), 5, dtype=dtype)
        bts = [_rand((n_local, k), 10 + r, 0.05, dtype=dtype) for r in range(world)]
        refs = [a.double() @ b.double().t() for b in bts]
        tols = [2.0 ** -9 * (a.double().abs() @ b.double().abs().t()) + 1e-6 for b in bts]
        same = [lambda got, want=want, tol=tol: bool(((got.double() - want).abs() <= tol).all())
                for want, tol in zip(refs, tols)]
    op = G.gemm_all_scatter(ranks, [a] * world, bts, push_kind=push_kind)
    for _ in range(3):
        outs = op()
    op.check()
    for r in range(world):
        assert outs[r].dtype == dtype
        for q in range(world):       # rank q's column block, as it arrived on rank r
            assert same[q](outs[r][:, q * n_local:(q + 1) * n_local]), (r, q)
    op.close()
    # all-gather prologue: every rank brings m / world rows of A, multiplies all m rows with its own B
    ag = G.all_gather_gemm(ranks, m, bts)
    ms = m // world
    for r in range(world):
        ag.a_full[r][r * ms:(r + 1) * ms].copy_(a[r * ms:(r + 1) * ms])
    for _ in range(2):
        outs = ag()
    ag.check()
    for r in range(world):
        assert same[r](outs[r]), r
    ag.close()
    ranks[0].close()


def test_fp32_int8_rejections():
    """The 32- and 8-bit types exist for the store mode with whole tiles; int8 tiles are 128 or 256 columns wide."""
    ctx = iris.Iris.local_world(1, heap_size=32 << 20)[0]
    a8, b8 = _int8_rand((256, 256), 1), _int8_rand((256, 256), 2)
    with pytest.raises(ValueError):
        G.FusedGemm(ctx, [a8], [b8], "store", bn=64)
    with pytest.raises(ValueError):
        G.FusedGemm(ctx, [a8], [b8], "reduce")
    af, bf = _rand((256, 256), 1, dtype=torch.float32), _rand((256, 256), 2, dtype=torch.float32)
    with pytest.raises(ValueError):
        G.FusedGemm(ctx, [af], [bf], "one_shot")
    with pytest.raises(ValueError):
        G.FusedGemm(ctx, [af], [bf], "store", stream_k=True)
    with pytest.raises(TypeError):
        G.FusedGemm(ctx, [af], [b8], "store")
    ctx.close()


@pytest.mark.parametrize("bn", [128, 256])
@pytest.mark.parametrize("m,n,k,cta_group", [(2560, 2048, 256, 2), (2560, 2048, 256, 1), (2816, 1800, 320, 2)])
def test_column_split_tail(m, n, k, cta_group, bn):
    """More tiles than scheduling units with a small ragged last wave: its tiles are cut into column pieces computed
    by different units (narrower MMAs, B fetched in narrower boxes).  Same result as the unsplit schedule, bit for bit."""
    a, bt = _rand((m, k), 3), _rand((n, k), 4, 0.05)
    ctx = iris.Iris.local_world(1, heap_size=64 << 20)[0]
    outs = []
    for split in (4, True, False):
        out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
        op = G.FusedGemm(ctx, [a], [bt], "store", out=[out], cta_group=cta_group, bn=bn, tail_split=split,
                         stream_k=False)   # (the default schedule would answer the ragged wave with stream-K)
        if split:
            assert op.tail_tiles > 0 and op.tail_split > 1, "shape does not exercise the split tail on this device"
        else:
            assert op.tail_tiles == 0
        for _ in range(2):
            op()
        op.check()
        _assert_close(out, a.float() @ bt.float().t())
        outs.append(out)
        op.close()
    assert torch.equal(outs[0], outs[2]) and torch.equal(outs[1], outs[2])
    ctx.close()


def test_many_tiles_per_cta_pair():
    # more tiles than CTA pairs: ring and accumulator phases wrap many times
    a, bt = _rand((4096, 512), 1), _rand((8192, 512), 2, 0.05)
    out = G.gemm(a, bt, cta_group=2)
    torch.cuda.synchronize()
    _assert_close(out, a.float() @ bt.float().t())


@pytest.mark.parametrize("m,n,k,cta_group", [(128, 4096, 1376, 1), (1, 4096, 1376, 1), (1024, 4096, 1376, 2),
                                               (2304, 2560, 2048, 2), (8192, 1792, 1024, 2), (640, 1280, 4160, 1)])
def test_stream_k_schedule(m, n, k, cta_group):
    """Tiles split by k-blocks across CTAs: the pieces that do not hold a tile's first k-blocks are parked as fp32 in
    workspace slots, the unit with the first k-blocks adds them to its accumulator and finishes the tile; called
    twice: the per-tile counters must be back at zero after every call."""
    a, bt = _rand((m, k), 1), _rand((n, k), 2, 0.05)
    ctx = iris.Iris.local_world(1, heap_size=256 << 20)[0]
    out = torch.zeros((m, n), dtype=torch.bfloat16, device="cuda")
    op = G.FusedGemm(ctx, [a], [bt], "store", out=[out], cta_group=cta_group, stream_k=True)
    assert op.sk_units > 0, "shape does not exercise the split schedule"
    for _ in range(2):
        out.zero_()
        op()
        op.check()
        _assert_close(out, a.float() @ bt.float().t())
    from iris_b200.ops.gemm_plan import FLAG_HEADER
    assert int(op.flags[0][FLAG_HEADER:].abs().sum()) == 0
    op.close()
    ctx.close()


def test_gemm_strided_views():
    # K-shards taken as views: row pitch larger than K, base offset inside the row
    big_a, big_b = _rand((512, 4096), 3), _rand((768, 4096), 4, 0.05)
    a, bt = big_a[:, 1376:2752], big_b[:, 1376:2752]
    out = G.gemm(a, bt)
    torch.cuda.synchronize()
    _assert_close(out, a.float() @ bt.float().t())


@pytest.mark.parametrize("push_kind", ["tma", "tma_spread", "stores"])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world,m,n_local,bn", [(2, 2560, 1024, 256), (4, 1000, 320, 128), (8, 512, 192, 64)])
def test_gemm_all_scatter_push_kinds(world, m, n_local, bn, dtype, push_kind):
    """Every way a finished tile travels to the other ranks (TMA stores from one or four issuing threads, 16-byte
    stores by all epilogue threads), with the column-split tail, narrower tiles, fp16 and a ragged M.  (The multimem
    form needs an NVLS-bound heap across real GPUs: tests/workers/gpu_vmm_nvls.py.)"""
    k = 384
    ranks = iris.Iris.local_world(world, heap_size=64 << 20)
    a = _rand((m, k), 5, dtype=dtype)
    bts = [_rand((n_local, k), 10 + r, 0.05, dtype=dtype) for r in range(world)]
    op = G.gemm_all_scatter(ranks, [a] * world, bts, bn=bn, push_kind=push_kind, tail_split=4)
    assert op.push_kind == push_kind
    for _ in range(3):
        outs = op()
    op.check()
    ref = torch.cat([a.float() @ b.float().t() for b in bts], dim=1)
    for r in range(world):
        _assert_close(outs[r], ref)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("stream_k", [False, True])
@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("world", [2, 4])
def test_gemm_all_scatter_emulated(world, cta_group, stream_k):
    m, n_local, k = 1024, 512, 512
    ranks = iris.Iris.local_world(world, heap_size=64 << 20)
    a = _rand((m, k), 5)
    bts = [_rand((n_local, k), 10 + r, 0.05) for r in range(world)]
    op = G.gemm_all_scatter(ranks, [a] * world, bts, cta_group=cta_group, stream_k=stream_k)
    for _ in range(3):  # cumulative flags must keep working call after call
        outs = op()
    op.check()
    ref = torch.cat([a.float() @ b.float().t() for b in bts], dim=1)
    for r in range(world):
        _assert_close(outs[r], ref)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("variant", ["atomic", "one_shot", "two_shot"])
@pytest.mark.parametrize("stream_k", [False, True])
@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("world", [2, 4])
def test_gemm_all_reduce_emulated(variant, world, cta_group, stream_k):
    m, n, k_full = 640, 768, 2752
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=64 << 20)
    a_full, b_full = _rand((m, k_full), 6), _rand((n, k_full), 7, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]       # views: pitch k_full
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    op = G.gemm_all_reduce(ranks, a, bt, variant=variant, cta_group=cta_group, stream_k=stream_k)
    for _ in range(3):
        outs = op()
    op.check()
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref = sum(parts)
    scale = sum(p.abs() for p in parts)
    for r in range(world):
        _assert_close(outs[r], ref, scale=scale, ulps=2.0 + world)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("variant", ["atomic", "one_shot", "two_shot", "reduce_scatter"])
@pytest.mark.parametrize("bn,dtype", [(128, torch.float16), (64, torch.bfloat16), (256, torch.float16)])
def test_collectives_in_fp16_and_narrow_tiles(variant, bn, dtype):
    """The reductions with fp16 operands (fp32 accumulation and summing) and with 64- / 128-column tiles."""
    world, m, n, k_full = 2, 1024, 832, 1408
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    a_full, b_full = _rand((m, k_full), 6, dtype=dtype), _rand((n, k_full), 7, 0.05, dtype=dtype)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    if variant == "reduce_scatter":
        op = G.gemm_reduce_scatter(ranks, a, bt, bn=bn)
    else:
        op = G.gemm_all_reduce(ranks, a, bt, variant=variant, bn=bn)
    for _ in range(3):
        outs = op()
    op.check()
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for r in range(world):
        rows = slice(r * m // world, (r + 1) * m // world) if variant == "reduce_scatter" else slice(0, m)
        assert outs[r].dtype == dtype
        _assert_close(outs[r], ref[rows], scale=scale[rows], ulps=2.0 + world)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("m,bn,ksplit", [(1, 64, 4), (128, 128, 8), (100, 256, 3), (256, 128, 2)])
@pytest.mark.parametrize("world", [2, 4])
def test_atomic_all_reduce_with_k_split(world, m, bn, ksplit):
    """Atomic all-reduce of a short matrix: every (tile, K piece) is computed by its own CTA and added straight into
    all ranks' outputs; called three times (the output is cleared before every call)."""
    n, k_full = 1024, 5504
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=96 << 20)
    a_full, b_full = _rand((m, k_full), 16), _rand((n, k_full), 17, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    op = G.gemm_all_reduce(ranks, a, bt, variant="atomic", bn=bn, ksplit=ksplit)
    assert op.ksplit == ksplit
    for _ in range(3):
        outs = op()
    op.check()
    # the partial sums are added up in bf16, piece by piece, in memory: the rounding acts on the pieces' magnitudes
    kb = -(-ks // 64)
    cuts = [min(ks, 64 * (kb * q // ksplit)) for q in range(ksplit + 1)]
    pieces = [a[r][:, cuts[q]:cuts[q + 1]].float() @ bt[r][:, cuts[q]:cuts[q + 1]].float().t()
              for r in range(world) for q in range(ksplit)]
    ref, scale = sum(pieces), sum(p.abs() for p in pieces)
    for r in range(world):
        _assert_close(outs[r], ref, scale=scale, ulps=2.0 + world * ksplit)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("m,ksplit", [(1, None), (100, None), (128, 3), (256, None), (128, 1)])
@pytest.mark.parametrize("world", [2, 4])
def test_one_shot_push_short_matrices(world, m, ksplit):
    """Short matrices: every rank's partial (per K piece) is pushed into an inbox slot of every rank and summed from
    local memory, the reducer work is split by column chunk."""
    n, k_full = 1024, 5504
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=96 << 20)
    a_full, b_full = _rand((m, k_full), 16), _rand((n, k_full), 17, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    op = G.gemm_all_reduce(ranks, a, bt, variant="one_shot", ksplit=ksplit)
    assert op.push
    for _ in range(3):
        outs = op()
    op.check()
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for r in range(world):
        _assert_close(outs[r], ref, scale=scale, ulps=2.0 + world * op.ksplit)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("world,m", [(2, 1024), (4, 2048), (4, 3072), (8, 2048)])
def test_gemm_reduce_scatter_emulated(world, m, cta_group):
    """GEMM + reduce-scatter: every rank keeps its own M / world rows of the sum; partial tiles go to the keeper only,
    in a rank-dependent order."""
    n, k_full = 768, 2048
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    a_full, b_full = _rand((m, k_full), 26), _rand((n, k_full), 27, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    op = G.gemm_reduce_scatter(ranks, a, bt, cta_group=cta_group)
    assert op.rs_rows == m // world
    for _ in range(3):
        outs = op()
    op.check()
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for r in range(world):
        rows = slice(r * op.rs_rows, (r + 1) * op.rs_rows)
        assert outs[r].shape == (op.rs_rows, n)
        _assert_close(outs[r], ref[rows], scale=scale[rows], ulps=2.0 + world)
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("world,m,cta_group,bn", [(2, 1024, 2, 256), (4, 2048, 2, 128), (4, 1536, 1, 256), (8, 2048, 2, 256),
                                                  (8, 1024, 1, 64)])
def test_push_two_shot_all_reduce_emulated(world, m, cta_group, bn, dtype):
    """GEMM + all-reduce as pushes only: partial tiles go to the keeper of their rows, the keeper sums them from local
    memory and writes the result rows into every rank's output."""
    n, k_full = 768, 2048
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    a_full, b_full = _rand((m, k_full), 26, dtype=dtype), _rand((n, k_full), 27, 0.05, dtype=dtype)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    op = G.gemm_all_reduce(ranks, a, bt, variant="two_shot_push", cta_group=cta_group, bn=bn)
    assert op.bcast and op.rs_rows == m // world
    for _ in range(3):
        outs = op()
    op.check()
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for r in range(world):
        assert outs[r].shape == (m, n)
        _assert_close(outs[r], ref, scale=scale, ulps=2.0 + world)
    op.close()
    ranks[0].close()


def test_no_kernel_writes_outside_its_buffers():
    """Every fused variant on a debug heap (guard bytes behind each allocation), shapes with ragged edges: after the
    calls the guards are intact and all ranks made the same allocations."""
    world = 2
    ranks = iris.Iris.local_world(world, heap_size=256 << 20, debug_heap=True)
    m, n, k_full = 648, 832, 1296          # M and N end inside a tile
    ks = k_full // world
    a_full, b_full = _rand((m, k_full), 41), _rand((n, k_full), 42, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    ops = [G.gemm_all_reduce(ranks, a, bt, variant=v) for v in ("atomic", "one_shot", "two_shot")]
    ops.append(G.gemm_all_reduce(ranks, [x[:100] for x in a], bt, variant="one_shot"))            # pushed, K-split
    ops.append(G.gemm_all_scatter(ranks, [a_full] * world, [_rand((320, k_full), 43 + r, 0.05) for r in range(world)]))
    ops.append(G.gemm_reduce_scatter(ranks, [x[:512] for x in a], bt))
    ops.append(G.gemm_all_reduce(ranks, [x[:512] for x in a], bt, variant="two_shot_push"))
    ag = G.all_gather_gemm(ranks, 512, [_rand((320, 512), 50 + r, 0.05) for r in range(world)], ag_slices=4)
    for r in range(world):
        ag.a_full[r][r * 256:(r + 1) * 256].copy_(_rand((256, 512), 60 + r))
    ops.append(ag)
    for _ in range(2):
        for op in ops:
            op()
    for op in ops:
        op.check()
    for r in ranks:
        r.barrier()      # checks guards and allocation sequences
    for op in ops:
        op.close()
    ranks[0].close()


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("world", [2, 4])
@pytest.mark.parametrize("n_local", [256, 1536])
def test_all_gather_gemm_emulated(world, cta_group, n_local):
    """n_local = 1536 gives more tiles than scheduling units with a ragged last wave and runs under the stream-K
    schedule (the default for larger problems of this kind), whose split tiles wait for their rows' chunk flags like
    whole tiles do."""
    m, k = 2048, 512
    ms = m // world
    ranks = iris.Iris.local_world(world, heap_size=256 << 20)
    a_full = _rand((m, k), 8)
    bts = [_rand((n_local, k), 20 + r, 0.05) for r in range(world)]
    op = G.all_gather_gemm(ranks, m, bts, ag_slices=4, cta_group=cta_group,
                           stream_k=True if n_local == 1536 else None)
    assert (op.sk_units > 0) == (n_local == 1536)
    for call in range(2):
        for r in range(world):  # every rank owns only its rows; the kernel gathers the rest
            op.a_full[r].zero_()
            op.a_full[r][r * ms:(r + 1) * ms].copy_(a_full[r * ms:(r + 1) * ms])
        outs = op()
        op.check()
        for r in range(world):
            assert torch.equal(op.a_full[r], a_full), f"gathered A differs on rank {r}"
            _assert_close(outs[r], a_full.float() @ bts[r].float().t())
    op.close()
    ranks[0].close()


@pytest.mark.parametrize("world", [2, 4])
def test_all_gather_gemm_back_to_back_calls_with_new_rows(world):
    """Calls follow one another on the stream with DIFFERENT rows and no host synchronisation in between: a rank
    must not write call k + 1's rows into a peer's gathered A while that peer still loads call k's (the entry-flag
    wait of the communication warps).  Every call's product is kept and checked at the end."""
    m, n_local, k, calls = 1024, 256, 512, 4
    ms = m // world
    ranks = iris.Iris.local_world(world, heap_size=64 << 20)
    bts = [_rand((n_local, k), 20 + r, 0.05) for r in range(world)]
    a_calls = [_rand((m, k), 70 + c) for c in range(calls)]
    op = G.all_gather_gemm(ranks, m, bts, ag_slices=4)
    kept = []
    for c in range(calls):
        for r in range(world):
            op.a_full[r][r * ms:(r + 1) * ms].copy_(a_calls[c][r * ms:(r + 1) * ms])
        outs = op()
        kept.append([o.clone() for o in outs])
    op.check()
    for c in range(calls):
        for r in range(world):
            _assert_close(kept[c][r], a_calls[c].float() @ bts[r].float().t())
    op.close()
    ranks[0].close()


def test_rebuild_after_a_reported_timeout_gives_a_working_op():
    """Recovery path on the host: a time-out record in a rank's status block (written here by the host, as a bounded
    wait of a kernel would) makes check() raise; rebuild() returns a fresh op that computes correctly.  (The device
    side of a time-out, a wait that runs out and returns, is exercised in test_gpu_rma.py.)"""
    world, m, n, k_full = 2, 640, 512, 1024
    ks = k_full // world
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    a_full, b_full = _rand((m, k_full), 6), _rand((n, k_full), 7, 0.05)
    a = [a_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    bt = [b_full[:, r * ks:(r + 1) * ks] for r in range(world)]
    parts = [a[r].float() @ bt[r].float().t() for r in range(world)]
    ref, scale = sum(parts), sum(p.abs() for p in parts)
    for variant in ("two_shot", "atomic"):
        op = G.gemm_all_reduce(ranks, a, bt, variant=variant)
        op()
        op.check()
        ranks[1].status[:4].copy_(torch.tensor([1, 32, 1, 7], dtype=torch.int32))   # code 1 = time-out, site, rank, tile
        with pytest.raises(iris.IrisTimeoutError):
            op.check()
        op2 = op.rebuild()
        assert op._plan is None and op2.calls == 0
        for _ in range(2):
            outs = op2()
        op2.check()
        for r in range(world):
            _assert_close(outs[r], ref, scale=scale, ulps=2.0 + world)
        op2.close()
    ranks[0].close()


def test_plan_rejects_bad_shapes():
    a, bt = _rand((128, 60), 1), _rand((256, 60), 2)
    with pytest.raises((RuntimeError, ValueError)):
        G.gemm(a, bt)


def test_fused_ops_replay_from_a_cuda_graph():
    """Launches carry no per-call argument (call number, flag targets and buffer parity live in device memory), so a
    stream capture records them once and the graph replays them: all-scatter, pulled and pushed all-reduce,
    reduce-scatter and the all-gather prologue, two ranks in one launch, with new inputs before every replay and
    ordinary calls mixed in."""
    world, m, n, k = 2, 512, 512, 512
    ranks = iris.Iris.local_world(world, heap_size=128 << 20)
    a = _rand((m, k), 1)
    bts = [_rand((n, k), 10 + r, 0.05) for r in range(world)]
    ks = k // world
    a_sh = [a[:, r * ks:(r + 1) * ks] for r in range(world)]
    b_sh = [bts[0][:, r * ks:(r + 1) * ks] for r in range(world)]
    ops = {
        "all_scatter": G.gemm_all_scatter(ranks, [a] * world, bts),
        "two_shot": G.gemm_all_reduce(ranks, a_sh, b_sh, variant="two_shot"),
        "one_shot": G.gemm_all_reduce(ranks, a_sh, b_sh, variant="one_shot"),
        "atomic": G.gemm_all_reduce(ranks, a_sh, b_sh, variant="atomic"),
        "reduce_scatter": G.gemm_reduce_scatter(ranks, a_sh, b_sh),
        "all_gather": G.all_gather_gemm(ranks, m, bts),
    }
    ms = m // world

    def fill_gathered():
        for r in range(world):
            ops["all_gather"].a_full[r][r * ms:(r + 1) * ms].copy_(a[r * ms:(r + 1) * ms])

    def run_all():
        fill_gathered()
        for op in ops.values():
            op()

    def verify():
        torch.cuda.synchronize()
        for op in ops.values():
            op.check()
        full = [a.float() @ b.float().t() for b in bts]
        parts = [a_sh[r].float() @ b_sh[r].float().t() for r in range(world)]
        red, scale = sum(parts), sum(p.abs() for p in parts)
        for r in range(world):
            _assert_close(ops["all_scatter"].out[r], torch.cat(full, dim=1))
            _assert_close(ops["all_gather"].out[r], full[r])
            for name in ("two_shot", "one_shot", "atomic"):
                _assert_close(ops[name].out[r], red, scale=scale, ulps=2.0 + world)
            _assert_close(ops["reduce_scatter"].out[r], red[r * ms:(r + 1) * ms], scale=scale[r * ms:(r + 1) * ms],
                          ulps=2.0 + world)

    run_all()                # an ordinary call first (odd call number)
    verify()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        run_all()
    for i in range(3):       # replays see even and odd call numbers, with new operands every time
        a.copy_(_rand((m, k), 100 + i))
        graph.replay()
        verify()
    a.copy_(_rand((m, k), 200))
    run_all()                # and ordinary calls keep working after replays
    verify()
    graph.replay()
    verify()
    for op in ops.values():
        op.close()
    ranks[0].close()
