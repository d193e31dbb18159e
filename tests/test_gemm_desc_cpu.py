"""``FusedGemm`` on a machine without a GPU: the real symmetric heap (CPU back end) under a stand-in for the kernel
library that records the descriptor and the launch arguments.  Checks the packing of the descriptor for every
collective, the buffer layout on the heap, and the cumulative per-call targets; and the pure planner
(``iris_b200/ops/gemm_plan.py``) over many shapes."""
import ctypes
from types import SimpleNamespace

import pytest
import torch

import iris_b200 as iris
from iris_b200.ops import gemm as G
from iris_b200.ops.gemm_plan import BM, FLAG_HEADER, plan_gemm


class FakeKernels:
    def __init__(self):
        self.descs, self.launches, self.destroyed = [], [], []

    def iris_gemm_plan_create(self, ref):
        self.descs.append(G._Desc.from_buffer_copy(bytes(ref._obj)))
        return len(self.descs)

    def iris_gemm_plan_ctas_per_rank(self, h):
        return self.descs[h - 1].ctas_per_rank

    def iris_gemm_plan_launch(self, h, stream):
        self.launches.append((h,))
        return 0

    def iris_gemm_plan_destroy(self, h):
        self.destroyed.append(h)

    def iris_gemm_last_error(self):
        return b""


@pytest.fixture()
def world2(monkeypatch):
    ranks = iris.Iris.local_world(2, heap_size=64 << 20, backend="cpu")
    fake = FakeKernels()
    monkeypatch.setattr(G, "_lib", lambda: fake)
    monkeypatch.setattr(torch.cuda, "get_device_properties", lambda dev: SimpleNamespace(multi_processor_count=148))
    for r in ranks:
        r.backend = "cuda"     # the op only asks; all memory stays on the CPU heap
    yield ranks, fake
    for r in ranks:
        r.backend = "cpu"
    ranks[0].close()


def _ab(m, n, k, world):
    a = [torch.zeros((m, k), dtype=torch.bfloat16) for _ in range(world)]
    bt = [torch.zeros((n, k), dtype=torch.bfloat16) for _ in range(world)]
    return a, bt


def test_all_scatter_descriptor(world2):
    ranks, fake = world2
    a, bt = _ab(512, 320, 256, 2)
    op = G.gemm_all_scatter(ranks, a, bt)
    d = fake.descs[-1]
    c0 = ranks[0]
    assert (d.M, d.N, d.K, d.world, d.num_local, d.rank0) == (512, 320, 256, 2, 2, 0)
    assert d.mode == G.MODES["store"] and d.store_all == 1 and d.cta_group == 2
    assert d.c_cols == 640 and d.col_off_per_rank == 320 and d.ldc == 640
    assert [d.c_ptr[t] for t in range(2)] == [c0.heap_base(t) + c0.offset_of(op.out[0]) for t in range(2)]
    assert d.flags_off == c0.offset_of(op.flags[0]) and d.status_off == c0.offset_of(c0.status)
    assert d.tile_flag_base == FLAG_HEADER and d.out_row0 == -1 and d.rs_rows == 0 and d.push_partials == 0
    assert [d.a_ptr[l] for l in range(2)] == [x.data_ptr() for x in a] and d.lda[0] == 256
    for _ in range(3):
        out = op(stream=0)
    assert out[0].shape == (512, 640)
    # a launch carries the plan and the stream only: the call number and what follows from it live in device memory
    assert fake.launches[-3:] == [(1,), (1,), (1,)] and op.calls == 3
    op.close()
    assert fake.destroyed == [1]


@pytest.mark.parametrize("variant", ["atomic", "one_shot", "two_shot"])
def test_all_reduce_descriptors(world2, variant):
    ranks, fake = world2
    a, bt = _ab(640, 768, 512, 2)
    op = G.gemm_all_reduce(ranks, a, bt, variant=variant)
    d, c0 = fake.descs[-1], ranks[0]
    if variant == "atomic":
        assert d.mode == G.MODES["reduce"] and d.store_all == 1 and d.out_row0 == -1
        assert d.c_ptr[1] == c0.heap_base(1) + c0.offset_of(op.out[0])
    else:
        mp = 768                                                  # 640 rows padded to whole 256-row tiles
        assert d.mode == G.MODES[variant] and d.push_partials == 0 and d.ksplit == 1
        assert (d.part_row0[0], d.part_row0[1], d.out_row0, d.c_rows) == (0, mp, 2 * mp, 3 * mp)
        assert c0.offset_of(op.out[0]) == c0.offset_of(op._pull_buf[0]) + 2 * mp * 768 * 2
        assert d.out_off == c0.offset_of(op.out[0]) and d.partial_off[0] == c0.offset_of(op._pull_buf[0])
        assert op.flags[0].numel() == FLAG_HEADER + op.total_tiles * op.cta_group
        op(stream=0), op(stream=0)
        assert fake.launches[-1] == (len(fake.descs),) and op.calls == 2
    assert op.out[0].shape == (640, 768)
    op.close()


def test_pushed_one_shot_and_reduce_scatter_descriptors(world2):
    ranks, fake = world2
    a, bt = _ab(100, 1024, 2048, 2)
    op = G.gemm_all_reduce(ranks, a, bt, variant="one_shot")     # short matrix: pushed, K split
    d = fake.descs[-1]
    assert op.push and op.ksplit > 1 and d.push_partials == 1 and d.ksplit == op.ksplit and d.cta_group == 1
    slots, mp = 2 * op.ksplit, 256
    assert d.part_slot_rows == mp and (d.part_row0[1], d.out_row0) == (slots * mp, 2 * slots * mp)
    op(stream=0)
    assert op.plan.flags_per_call == 2 * op.ksplit                # every (rank, piece) arrives once per call
    op.close()
    a, bt = _ab(1024, 512, 256, 2)
    rs = G.gemm_reduce_scatter(ranks, a, bt)
    d = fake.descs[-1]
    assert d.rs_rows == 512 and d.push_partials == 1 and d.ksplit == 1 and d.mode == G.MODES["one_shot"]
    assert d.part_slot_rows == 512 and d.c_rows == (2 * 2 + 1) * 512 and d.group_m == 2   # 2 m-tiles per keeper
    assert rs.out[0].shape == (512, 512) and rs.out[1].shape == (512, 512)
    with pytest.raises(ValueError, match="multiple of world"):
        G.gemm_reduce_scatter(ranks, [x[:1000] for x in a], bt)
    rs.close()


def test_all_gather_gemm_descriptor(world2):
    ranks, fake = world2
    bt = [torch.zeros((256, 512), dtype=torch.bfloat16) for _ in range(2)]
    op = G.all_gather_gemm(ranks, 1024, bt, ag_slices=4)
    d, c0 = fake.descs[-1], ranks[0]
    assert d.ag == 1 and d.ag_slices == 4 and d.agsrc_off == c0.offset_of(op.a_full[0]) and d.cta_group == 1
    assert d.ag_flag_base == FLAG_HEADER and op.flags[0].numel() == FLAG_HEADER + 2 * (512 // BM)
    assert d.a_ptr[1] == op.a_full[1].data_ptr()
    op.close()


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_planner_invariants(world):
    import random
    rnd = random.Random(world)
    for _ in range(3000):
        mode = rnd.choice(["store", "reduce", "one_shot", "two_shot"])
        M = rnd.choice([1, 100, 128, 129, 640, 1024, 8192, rnd.randint(1, 20000)])
        N = 8 * rnd.randint(1, 2000)
        K = 8 * rnd.randint(1, 2000)
        nl = rnd.choice([1, world])
        p = plan_gemm(M, N, K, world, nl, mode, 148, stream_k=rnd.choice([False, True]),
                      cta_group=rnd.choice([None, 1, 2]), store_all=True)
        assert p.ctas_per_rank >= p.cta_group and p.ctas_per_rank % p.cta_group == 0
        assert p.ctas_per_rank * nl <= 148
        assert p.total_tiles == -(-M // (BM * p.cta_group)) * -(-N // 256)
        assert 0 <= p.dp_tiles <= p.total_tiles and p.dp_tiles + p.sk_tiles == p.total_tiles
        assert (p.sk_units > 0) == (p.sk_tiles > 0)
        assert p.ksplit >= 1 and (p.ksplit == 1 or p.push) and (not p.push or mode == "one_shot")
        assert p.nflags == FLAG_HEADER + p.tile_flags + p.sk_flags
        if p.pulls:
            assert p.slot_rows % 256 == 0 and p.slot_rows >= p.rows == M
            assert p.part_row0 == (0, p.slots * p.slot_rows) and p.out_row0 == 2 * p.slots * p.slot_rows
            assert p.c_rows == p.regions * p.slot_rows and p.slots == (world * p.ksplit if p.push else 1)
            assert p.world * p.ksplit <= 16 or not p.push or p.ksplit == 1
        assert p.store_all == (world > 1)


def test_planner_named_configurations():
    p = plan_gemm(8192, 1792, 4096, 8, 1, "store", 148, store_all=True)          # GEMM + all-scatter, 8 ranks
    assert (p.cta_group, p.ctas_per_rank, p.total_tiles, p.kblocks) == (2, 148, 224, 64)
    p = plan_gemm(8192, 1792, 4096, 1, 1, "store", 148)                          # the same shape kept local: single CTAs
    assert (p.cta_group, p.total_tiles) == (1, 448)
    p = plan_gemm(8192, 14336, 4096, 1, 1, "store", 148, group_m=None)           # the whole product on one GPU
    assert (p.cta_group, p.ctas_per_rank, p.total_tiles, p.group_m) == (2, 148, 1792, 16)
    p = plan_gemm(8192, 4096, 1376, 8, 1, "two_shot", 148)                       # GEMM + all-reduce, 8 ranks
    assert (p.cta_group, p.total_tiles, p.tile_flags, p.slot_rows, p.regions) == (2, 512, 1024, 8192, 3)
    p = plan_gemm(1, 4096, 1376, 8, 1, "one_shot", 148)                          # one row: pushed, K in 2 pieces
    assert (p.cta_group, p.push, p.ksplit, p.ctas_per_rank, p.slots) == (1, True, 2, 32, 16)
    p = plan_gemm(16384, 4096, 512, 8, 1, "one_shot", 148, reduce_scatter=True)  # row-parallel projection, 8 ranks
    assert (p.rs_rows, p.group_m, p.slots, p.slot_rows, p.c_rows) == (2048, 8, 8, 2048, 17 * 2048)
    with pytest.raises(ValueError):
        plan_gemm(1024, 256, 256, 2, 1, "two_shot", 148, reduce_scatter=True)
    with pytest.raises(ValueError):
        plan_gemm(1024, 256, 256, 2, 1, "one_shot", 148, ag=True)


def test_new_plan_knobs_reach_the_descriptor(world2):
    """Tile width, element type, push kind, column-split tail, K pieces of the atomic form and the push two-shot
    layout, as the native library receives them."""
    ranks, fake = world2
    a = [torch.zeros((2560, 256), dtype=torch.float16) for _ in range(2)]
    bt = [torch.zeros((1024, 256), dtype=torch.float16) for _ in range(2)]
    op = G.gemm_all_scatter(ranks, a, bt, bn=128, push_kind="stores", tail_split=2)
    d, c0 = fake.descs[-1], ranks[0]
    assert (d.bn, d.dtype, d.push_kind) == (128, G.DTYPES["fp16"], G.PUSH_KINDS["stores"])
    assert d.c_off == c0.offset_of(op.out[0]) and op.out[0].dtype == torch.float16
    # 10 x 8 = 80 pair-tiles on 37 units: 2 full waves, 6 tiles left -> cut in two column pieces each
    assert (d.tail_tiles, d.tail_split) == (6, 2) == (op.tail_tiles, op.tail_split)
    op.close()
    with pytest.raises(RuntimeError, match="multimem"):
        G.gemm_all_scatter(ranks, a, bt, push_kind="multimem")     # no NVLS-bound heap on this machine
    with pytest.raises(TypeError):
        G.gemm_all_scatter(ranks, a, [b.to(torch.bfloat16) for b in bt])   # mixed element types
    a, bt = _ab(128, 1024, 2048, 2)
    at = G.gemm_all_reduce(ranks, a, bt, variant="atomic", bn=64, ksplit=4)
    d = fake.descs[-1]
    assert (d.mode, d.ksplit, d.bn, d.store_all) == (G.MODES["reduce"], 4, 64, 1) and at.ctas_per_rank == 64
    at.close()
    a, bt = _ab(1024, 512, 256, 2)
    tp = G.gemm_all_reduce(ranks, a, bt, variant="two_shot_push")
    d = fake.descs[-1]
    assert d.rs_rows == 512 and d.rs_bcast == 1 and d.push_partials == 1
    # inbox: 2 parities x 2 slots of 512 rows; output: all 1024 rows on every rank
    assert d.c_rows == (2 * 2 + 2) * 512 and d.out_row0 == 4 * 512 and tp.out[0].shape == (1024, 512)
    tp2 = tp.rebuild()
    assert tp._plan is None and fake.descs[-1].rs_bcast == 1 and tp2.calls == 0
    tp2.close()


def test_auto_variant_table():
    assert G.auto_all_reduce_variant(1, 8) == ("atomic", dict(bn=128, ksplit=4))
    assert G.auto_all_reduce_variant(128, 8) == ("atomic", dict(bn=64))
    assert G.auto_all_reduce_variant(1, 2)[0] == "atomic" and G.auto_all_reduce_variant(1, 2)[1]["ksplit"] == 8
    assert G.auto_all_reduce_variant(1024, 2)[0] == "one_shot"
    assert G.auto_all_reduce_variant(8192, 8)[0] == "two_shot" and G.auto_all_reduce_variant(1024, 4)[0] == "two_shot"


def test_planner_element_types():
    """K slices and epilogue sub-tiles are 128 bytes whatever the element: 64 / 32 / 128 elements for 16- / 32- / 8-bit
    types; the 32- and 8-bit types are store-mode only."""
    kw = dict(world=1, num_local=1, mode="store", sms=148)
    assert plan_gemm(1024, 1024, 4096, dtype="bf16", **kw).kblocks == 64
    assert plan_gemm(1024, 1024, 4096, dtype="fp32", **kw).kblocks == 128
    assert plan_gemm(1024, 1024, 4096, dtype="int8", **kw).kblocks == 32
    assert plan_gemm(1024, 1024, 4096, dtype="fp32", bn=64, **kw).bn == 64
    with pytest.raises(ValueError):
        plan_gemm(1024, 1024, 4096, dtype="int8", bn=64, **kw)
    for bad in (dict(mode="reduce"), dict(mode="one_shot"), dict(mode="two_shot"), dict(stream_k=True)):
        args = dict(kw)
        args.update(bad)
        with pytest.raises(ValueError):
            plan_gemm(1024, 1024, 4096, dtype="int8", **args)
    with pytest.raises(ValueError):
        plan_gemm(1024, 1024, 4096, dtype="fp64", **kw)
    # a tail piece is a whole number of sub-tiles: int8 tiles of 256 columns split into two at most
    p = plan_gemm(2560, 2048, 256, dtype="int8", tail_split=4, ctas_per_rank=148, cta_group=1, **kw)
    assert p.tail_split in (1, 2)


def test_stream_k_default_rule(monkeypatch):
    """Stream-K is the default exactly where it was measured to pay: store / reduce kernels, 16-bit elements, at least
    one full wave of whole tiles before a ragged last one, and (with tiles pushed to peers) compute time above push
    time.  `stream_k=` and the environment variable IRIS_STREAM_K override it."""
    monkeypatch.delenv("IRIS_STREAM_K", raising=False)
    one = dict(world=1, num_local=1, mode="store", sms=148)
    assert plan_gemm(8192, 3584, 4096, **one).sk_units > 0              # 6.05 waves of single-CTA tiles
    assert plan_gemm(8192, 14336, 4096, **one).sk_units > 0             # 24.2 waves of pair tiles
    p = plan_gemm(8192, 14336, 4096, **one)
    assert p.dp_tiles % (p.ctas_per_rank // p.cta_group) == 0 and p.sk_tiles == p.total_tiles - p.dp_tiles
    assert p.sk_slots == 1                                              # ranges longer than a tile: one parked piece
    assert plan_gemm(1024, 8192, 8192, **one).sk_units == 0             # fewer than two waves: every tile would split
    assert plan_gemm(2048, 2048, 8192, **one).sk_units == 0             # fewer tiles than units
    assert plan_gemm(8192, 5120, 4096, **one).sk_units == 0             # last wave 0.65 full: nothing to gain
    assert plan_gemm(8192, 3584, 4096, dtype="int8", **one).sk_units == 0
    assert plan_gemm(8192, 3584, 4096, stream_k=False, **one).sk_units == 0
    for mode in ("one_shot", "two_shot"):
        assert plan_gemm(8192, 4096, 1376, world=8, num_local=1, mode=mode, sms=148).sk_units == 0
    # tiles pushed to peers: on while the MMAs set the time (2 ranks), off where the pushes do (4 and 8 ranks)
    assert plan_gemm(8192, 7168, 4096, world=2, num_local=1, mode="store", sms=148, store_all=True).sk_units > 0
    assert plan_gemm(8192, 3584, 4096, world=4, num_local=1, mode="store", sms=148, store_all=True).sk_units == 0
    assert plan_gemm(8192, 1792, 4096, world=8, num_local=1, mode="store", sms=148, store_all=True).sk_units == 0
    # the all-gather prologue keeps the default (tiles wait for their rows either way)
    assert plan_gemm(16384, 3072, 4096, world=2, num_local=1, mode="store", sms=148, ag=True).sk_units > 0
    monkeypatch.setenv("IRIS_STREAM_K", "0")
    assert plan_gemm(8192, 3584, 4096, **one).sk_units == 0
    monkeypatch.setenv("IRIS_STREAM_K", "1")
    assert plan_gemm(1024, 8192, 8192, **one).sk_units > 0
    assert plan_gemm(8192, 3584, 4096, stream_k=False, **one).sk_units == 0   # an explicit argument wins
