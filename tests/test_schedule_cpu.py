"""Invariants of the fused GEMM's tile schedules, checked on the host through the C wrappers of the very functions
the kernel calls (iris_b200/csrc/kernels/gemm_schedule.h).  The reference has its schedule arithmetic inline in the
Triton kernels (examples/07_gemm_all_scatter/gemm_all_scatter.py:158-163 for the grouped raster) and no test of it."""
import ctypes
import itertools

import pytest

from iris_b200 import _build


@pytest.fixture(scope="module")
def lib():
    so = ctypes.CDLL(str(_build.build_all()["kernels"]))
    so.iris_sched_raster.argtypes = [ctypes.c_int] * 4 + [ctypes.POINTER(ctypes.c_int)] * 2
    so.iris_sched_raster.restype = None
    so.iris_sched_work_list.argtypes = [ctypes.c_int] * 7 + [ctypes.POINTER(ctypes.c_int), ctypes.c_int]
    so.iris_sched_work_list.restype = ctypes.c_int
    for f in (so.iris_sched_ag_actual_m, so.iris_sched_two_shot_owner, so.iris_sched_rs_tile_of):
        f.argtypes = [ctypes.c_int] * (3 if f is so.iris_sched_two_shot_owner else 4)
        f.restype = ctypes.c_int
    return so


def _raster(lib, t, tm, tn, g):
    m, n = ctypes.c_int(), ctypes.c_int()
    lib.iris_sched_raster(t, tm, tn, g, ctypes.byref(m), ctypes.byref(n))
    return m.value, n.value


@pytest.mark.parametrize("tm,tn,g", [(1, 1, 8), (32, 56, 8), (5, 3, 8), (13, 7, 4), (64, 16, 8), (7, 1, 2), (3, 9, 1)])
def test_grouped_raster_is_a_bijection_onto_the_tile_grid(lib, tm, tn, g):
    seen = {_raster(lib, t, tm, tn, g) for t in range(tm * tn)}
    assert seen == set(itertools.product(range(tm), range(tn)))
    # consecutive tiles of a full group walk down the group's m-tiles first
    if tm >= g:
        assert [_raster(lib, t, tm, tn, g)[0] for t in range(g)] == list(range(g))
        assert {_raster(lib, t, tm, tn, g)[1] for t in range(g)} == {0}


@pytest.mark.parametrize("world,per_shard", [(2, 4), (4, 2), (8, 1), (8, 8)])
def test_all_gather_order_starts_with_own_rows_and_is_a_permutation(lib, world, per_shard):
    for rank in range(world):
        order = [lib.iris_sched_ag_actual_m(m, per_shard, rank, world) for m in range(world * per_shard)]
        assert sorted(order) == list(range(world * per_shard))
        assert order[:per_shard] == list(range(rank * per_shard, (rank + 1) * per_shard))
        # then the peers in ring order: shard position sp holds the rows of rank (rank + sp) % world
        for sp in range(world):
            assert order[sp * per_shard] // per_shard == (rank + sp) % world


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("units,tiles", [(74, 512), (74, 1024), (148, 448), (37, 100)])
def test_two_shot_owner_gives_every_unit_the_same_share(lib, world, units, tiles):
    """Unit u visits tiles u, u + units, ...; of those, the ones it must also sum (owner == its rank) differ by at most
    one between any two (unit, rank) pairs, and every tile has exactly one owner."""
    share = {}
    for t in range(tiles):
        o = lib.iris_sched_two_shot_owner(t, units, world)
        assert 0 <= o < world
        share[(t % units, o)] = share.get((t % units, o), 0) + 1
    counts = [share.get((u, r), 0) for u in range(min(units, tiles)) for r in range(world)]
    visits = -(-tiles // units)
    assert max(counts) - min(counts) <= 1 + (visits % world != 0)
    assert max(counts) <= -(-visits // world)


@pytest.mark.parametrize("world,tpb", [(1, 16), (2, 512), (4, 6), (8, 128), (8, 1)])
def test_reduce_scatter_order(lib, world, tpb):
    total = world * tpb
    per_rank = [[lib.iris_sched_rs_tile_of(i, r, world, tpb) for i in range(total)] for r in range(world)]
    for r in range(world):
        assert sorted(per_rank[r]) == list(range(total))          # every rank computes every tile once
    for i in range(total):
        keepers = [per_rank[r][i] // tpb for r in range(world)]
        assert sorted(keepers) == list(range(world))              # one sender per keeper at every step
        assert keepers[0] == (1 + i) % world
    for r in range(world):
        for j in range(tpb):
            for b in range(world):                                 # tile j of block b is done after (j + 1) * world steps
                assert per_rank[r].index(b * tpb + j) < (j + 1) * world
    if world > 1:
        assert per_rank[0][0] // tpb == 1 and per_rank[0][world - 1] // tpb == 0   # next rank first, own block last


def _work(lib, unit, units, tiles, kblocks, dp_tiles, sk_units, ksplit):
    cap = 4096
    buf = (ctypes.c_int * (4 * cap))()
    n = lib.iris_sched_work_list(unit, units, tiles, kblocks, dp_tiles, sk_units, ksplit, buf, cap)
    assert n <= cap
    return [tuple(buf[4 * i:4 * i + 4]) for i in range(n)]


@pytest.mark.parametrize("m,n,k,world,mode,kw", [
    (8192, 1792, 4096, 8, "store", {}),                                  # whole tiles only
    (8192, 1792, 4096, 8, "store", {"stream_k": True}),                  # ragged last wave split by k-blocks
    (640, 768, 1376, 2, "one_shot", {"stream_k": True, "cta_group": 1}),
    (300, 520, 200, 1, "store", {"stream_k": True}),
    (128, 4096, 1376, 8, "one_shot", {}),                                # pushed, K split into pieces
    (1, 1024, 5504, 2, "one_shot", {"ksplit": 3}),
    (100, 4096, 64, 4, "one_shot", {}),                                  # one k-block: no split possible
])
def test_every_k_block_of_every_tile_is_computed_exactly_once(lib, m, n, k, world, mode, kw):
    """Over all scheduling units: whole tiles, stream-K ranges and K-split pieces together cover each (tile, k-block)
    once; a K-split tile has exactly `ksplit` pieces, which partition its k-blocks in order."""
    from iris_b200.ops.gemm_plan import plan_gemm
    p = plan_gemm(m, n, k, world, 1, mode, 148, **kw)
    units = p.ctas_per_rank // p.cta_group
    dp = p.dp_tiles if p.sk_units else p.total_tiles       # what FusedGemm hands to the kernel (-1 = all whole)
    seen = {}
    pieces = {}
    for u in range(units):
        for tile, kb0, kb1, piece in _work(lib, u, units, p.total_tiles, p.kblocks, dp, p.sk_units, p.ksplit):
            assert 0 <= tile < p.total_tiles and 0 <= kb0 < kb1 <= p.kblocks
            for kb in range(kb0, kb1):
                assert (tile, kb) not in seen, f"k-block {kb} of tile {tile} computed by units {seen[(tile, kb)]} and {u}"
                seen[(tile, kb)] = u
            pieces.setdefault(tile, []).append((piece, kb0, kb1))
    assert len(seen) == p.total_tiles * p.kblocks
    if p.ksplit > 1:
        for tile, ps in pieces.items():
            ps.sort()
            assert [q[0] for q in ps] == list(range(p.ksplit))
            assert ps[0][1] == 0 and ps[-1][2] == p.kblocks and all(a[2] == b[1] for a, b in zip(ps, ps[1:]))
    if kw.get("stream_k") and p.sk_units:
        # stream-K: the units' shares of the split part differ by at most one k-block
        share = [0] * units
        for (tile, kb), u in seen.items():
            if tile >= p.dp_tiles:
                share[u] += 1
        used = [x for x in share[:p.sk_units]]
        assert max(used) - min(used) <= 1 and sum(share[p.sk_units:]) == 0


@pytest.mark.parametrize("tiles,units,max_split", [(1792, 74, 4), (896, 74, 4), (448, 74, 4), (224, 74, 4), (300, 148, 2),
                                                   (75, 74, 4), (74, 74, 4), (50, 74, 4), (200, 74, 1), (1776, 74, 4)])
def test_column_split_tail_covers_every_piece_once_and_balances_the_last_wave(lib, tiles, units, max_split):
    """The ragged last wave is cut into column pieces: the native rule and the Python planner agree, every whole tile
    and every (tail tile, column piece) is visited exactly once, and no unit gets more than one piece of the tail."""
    from iris_b200.ops.gemm_plan import tail_split_plan
    lib.iris_sched_tail_split.argtypes = [ctypes.c_int] * 3 + [ctypes.POINTER(ctypes.c_int)] * 2
    lib.iris_sched_tail_split.restype = None
    lib.iris_sched_work_list_tail.argtypes = [ctypes.c_int] * 9 + [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int]
    lib.iris_sched_work_list_tail.restype = ctypes.c_int
    tt, sp = ctypes.c_int(), ctypes.c_int()
    lib.iris_sched_tail_split(tiles, units, max_split, ctypes.byref(tt), ctypes.byref(sp))
    assert (tt.value, sp.value) == tail_split_plan(tiles, units, max_split)
    tail, split = tt.value, sp.value
    if tiles % units and 2 * (tiles % units) <= units and tiles > units and max_split > 1:
        assert tail == tiles % units and split > 1 and tail * split <= units
    else:
        assert (tail, split) == (0, 1)
    kblocks, seen, per_unit_tail = 7, {}, []
    for u in range(units):
        buf = (ctypes.c_int * (6 * 64))()
        n = lib.iris_sched_work_list_tail(u, units, tiles, kblocks, tiles, 0, 1, tail, split, buf, 64, 6)
        assert n <= 64
        items = [tuple(buf[6 * i:6 * i + 6]) for i in range(n)]
        per_unit_tail.append(sum(1 for it in items if it[5] > 1))
        for tile, kb0, kb1, piece, sub, nsub in items:
            assert (kb0, kb1, piece) == (0, kblocks, 0)
            assert (tile >= tiles - tail) == (nsub > 1) and 0 <= sub < nsub and nsub in (1, split)
            seen[(tile, sub)] = seen.get((tile, sub), 0) + 1
    want = {(t, 0) for t in range(tiles - tail)} | {(t, s) for t in range(tiles - tail, tiles) for s in range(split)}
    assert set(seen) == want and set(seen.values()) == {1}
    assert max(per_unit_tail) <= 1
    # the whole tiles before the tail are whole waves: every unit has the same number of them
    if tail:
        assert (tiles - tail) % units == 0


@pytest.mark.parametrize("m,n,k,cta_group", [(4096, 4096, 4096, 2), (4096, 4096, 4096, 1), (128, 4096, 1376, 1),
                                             (1, 4096, 1376, 1), (1024, 8192, 8192, 2), (2304, 2560, 2048, 2),
                                             (640, 1280, 4160, 1), (8192, 1792, 1024, 2), (300, 520, 200, 1)])
def test_stream_k_pieces_know_their_slot_and_finisher(lib, m, n, k, cta_group):
    """What the epilogue derives from `sk_unit_of`: the piece with a tile's first k-blocks is the last item of its unit's
    range and expects exactly the tile's other pieces; those are computed by the following units, each the first item
    of its range unless the range lies inside one tile, and their slots are 0 .. kSkSlots - 1 without repeats."""
    from iris_b200.ops.gemm_plan import SK_SLOTS, plan_gemm
    assert lib.iris_sched_sk_slots() == SK_SLOTS
    lib.iris_sched_sk_unit_of.argtypes = [ctypes.c_longlong, ctypes.c_longlong, ctypes.c_int]
    p = plan_gemm(m, n, k, 1, 1, "store", 148, stream_k=True, cta_group=cta_group)
    if not p.sk_units:
        pytest.skip("no ragged wave on this shape")
    units = p.ctas_per_rank // p.cta_group
    S = (p.total_tiles - p.dp_tiles) * p.kblocks
    split = {}
    for u in range(units):
        items = _work(lib, u, units, p.total_tiles, p.kblocks, p.dp_tiles, p.sk_units, 1)
        sk = [it for it in items if it[0] >= p.dp_tiles]
        for i, (tile, kb0, kb1, _) in enumerate(sk):
            if kb0 == 0 and kb1 == p.kblocks:
                continue
            t = tile - p.dp_tiles
            head = lib.iris_sched_sk_unit_of(t * p.kblocks, S, p.sk_units)
            last = lib.iris_sched_sk_unit_of((t + 1) * p.kblocks - 1, S, p.sk_units)
            rec = split.setdefault(tile, dict(head=head, last=last, slots=[], finisher=None))
            assert (rec["head"], rec["last"]) == (head, last)
            if kb0 == 0:
                assert u == head and i == len(sk) - 1, "the finisher's piece must close its unit's range"
                rec["finisher"] = u
            else:
                assert head < u <= last
                rec["slots"].append(u - head - 1)
    assert split, "shape does not exercise split tiles"
    for tile, rec in split.items():
        assert rec["finisher"] == rec["head"]
        assert sorted(rec["slots"]) == list(range(rec["last"] - rec["head"])), (tile, rec)
        assert len(rec["slots"]) <= SK_SLOTS
