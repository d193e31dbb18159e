"""Schedule and buffer layout of one fused GEMM + collective, as a pure function of the problem: no device, no
allocation.  ``FusedGemm`` builds its kernel descriptor from the result; tests exercise it on a machine without a GPU.

Role in the reference: the Stream-K bookkeeping of ``examples/07_gemm_all_scatter/matmul_wrapper.py:63-103`` (tiles,
full waves, split tiles) and the buffer set-up of ``examples/09_gemm_one_shot_all_reduce/benchmark.py:103-142``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass
from typing import Optional, Tuple

BM, BN, BK = 128, 256, 64   # rows per CTA, widest tile in columns, k-block; the tile width is a launch parameter
TILE_WIDTHS = (64, 128, 256)
MODES = {"store": 0, "reduce": 1, "one_shot": 2, "two_shot": 3}
PUSH_KINDS = {"tma": 0, "tma_spread": 1, "stores": 2, "multimem": 3}
DTYPES = {"bf16": 0, "fp16": 1, "fp32": 2, "int8": 3}   # ElemType of the kernel; fp32 is multiplied as tf32
ELEM_BYTES = {"bf16": 2, "fp16": 2, "fp32": 4, "int8": 1}
SK_SLOTS = 3                # workspace slots per split tile part (kSkSlots of gemm_schedule.h)
FLAG_HEADER = 16            # flag words [0] arrival counter, [8 + r] entry flag of rank r; per-tile flags follow


@dataclass(frozen=True)
class GemmPlan:
    M: int
    N: int
    K: int
    world: int
    num_local: int
    mode: str
    ag: bool
    cta_group: int          # 1: one CTA per 128 x 256 tile; 2: a CTA pair per 256 x 256 tile
    group_m: int            # raster: m-tiles per group
    rs_rows: int            # reduce-scatter: rows kept per rank (0: off)
    ctas_per_rank: int      # CTAs asked for (the native plan may lower it to what is resident at once)
    total_tiles: int
    kblocks: int
    dp_tiles: int           # tiles computed whole; the rest is split by k-blocks (stream-K)
    sk_units: int
    sk_tiles: int
    push: bool              # one-shot: partials pushed into inbox slots
    ksplit: int             # pieces of K computed by different CTAs (push only)
    store_all: bool
    pulls: bool             # one-/two-shot family: partial buffers, per-tile flags, reducer warps
    chunks_per_shard: int   # all-gather prologue: 128-row chunks per rank
    tile_flags: int
    sk_flags: int
    nflags: int
    # layout of the [partials | out] matrix of the one-/two-shot family (rows; 0 / -1 when unused)
    rows: int               # rows of one slot and of the output
    slot_rows: int          # the same, padded to whole 256-row tiles
    slots: int              # inbox slots per parity
    regions: int
    c_rows: int
    part_row0: Tuple[int, int]
    out_row0: int
    out_rows: int = 0       # rows of the output region (M for the push two-shot, else `rows`)
    bcast: bool = False     # reduce-scatter whose keeper broadcasts the summed rows (push two-shot all-reduce)
    bn: int = BN            # tile width in columns
    tail_tiles: int = 0     # tiles at the end of the raster that are cut into column pieces ...
    tail_split: int = 1     # ... and into how many (1: none)
    sk_slots: int = 0       # stream-K: workspace slots per split tile part (the units a tile meets, less the finisher)

    @property
    def flags_per_call(self) -> int:
        """What one call adds to a per-tile flag (arrivals from all ranks and pieces)."""
        return self.world * self.ksplit


def sk_unit_of(x: int, S: int, U: int) -> int:
    """The unit whose stream-K range holds iteration ``x`` when ``S`` iterations are cut into ``U`` ranges with
    boundaries ``S * i // U`` (``sk_unit_of`` of ``csrc/kernels/gemm_schedule.h``)."""
    return ((x + 1) * U - 1) // S


def tail_split_plan(total_tiles: int, units: int, max_split: int) -> Tuple[int, int]:
    """``(tail_tiles, split)``: the ragged last wave of ``total_tiles`` on ``units`` scheduling units is cut into
    column pieces when it fills at most half of the units (the same rule as ``tail_split_plan`` in
    ``csrc/kernels/gemm_schedule.h``; the reference's persistent loop has the ragged wave and nothing against it,
    ``examples/07_gemm_all_scatter/gemm_all_scatter.py:153``)."""
    if units < 1 or total_tiles <= units:
        return 0, 1
    r = total_tiles % units
    if r == 0 or 2 * r > units:
        return 0, 1
    s, c = 1, 2
    while c <= max_split:
        if max_split % c == 0 and r * c <= units:
            s = c
        c *= 2
    return (r, s) if s > 1 else (0, 1)


def plan_gemm(M: int, N: int, K: int, world: int, num_local: int, mode: str, sms: int, *, ag: bool = False,
              cta_group: Optional[int] = None, ctas_per_rank: Optional[int] = None, group_m: Optional[int] = 8,
              stream_k: Optional[bool] = None, push: Optional[bool] = None, ksplit: Optional[int] = None,
              reduce_scatter: bool = False, store_all: bool = False, own_out: bool = False,
              bn: Optional[int] = None, tail_split: Optional[bool] = None, bcast: bool = False,
              dtype: str = "bf16") -> GemmPlan:
    """Decide tile shape, persistent grid, schedule, flag count and buffer layout.  ``sms``: SMs of the device;
    ``own_out``: the caller brings the output buffer (the [partials | out] matrix then has no output region);
    ``bn``: tile width (64, 128 or 256; default 256); ``tail_split``: cut the tiles of a ragged last wave into column
    pieces: ``True`` = into two, an integer = into at most that many (store / reduce modes with whole tiles; default
    off: measured on the 8192 x 14336 x 4096 problem the narrower pieces re-read A and lose more than the ragged wave
    costs); ``dtype``: element type of A, B and C (``DTYPES``); the 32- and 8-bit types exist for mode ``"store"``
    with whole tiles, and their tiles are a multiple of 32 / 128 columns wide (one 128-byte row of output per
    sub-tile)."""
    if mode not in MODES:
        raise ValueError(f"mode must be one of {sorted(MODES)}")
    bn = BN if bn is None else int(bn)
    if bn not in TILE_WIDTHS:
        raise ValueError(f"tile width must be one of {TILE_WIDTHS}")
    if dtype not in DTYPES:
        raise ValueError(f"dtype must be one of {sorted(DTYPES)}")
    es = ELEM_BYTES[dtype]
    sub_cols = 128 // es                     # output columns of one epilogue sub-tile; also K elements per ring stage
    if bn % sub_cols:
        raise ValueError(f"{dtype}: the tile width must be a multiple of {sub_cols} columns")
    if es != 2 and (mode != "store" or stream_k or reduce_scatter or (ksplit or 1) > 1):
        raise ValueError(f"{dtype} matrices: mode 'store' with whole tiles only (plain GEMM, all-scatter, all-gather)")
    if mode in ("one_shot", "two_shot") and ag:
        raise ValueError("the all-gather prologue is combined with mode='store' only")
    # CTA pairs (256-row tiles, cta_group::2) or single CTAs (128-row tiles).  Measured on 8192 x N x 4096: the pair
    # wins only when there are many column tiles (N = 14336: 658 us against 675 us); at N = 7168 / 3584 / 1792 single
    # CTAs are 3 to 7 % faster (343 / 185 / 107 us against 358 / 196 / 115 us), so the kernels that keep their tiles
    # (plain GEMM, all-gather -> GEMM) use pairs only above 8192 columns.  The one- / two-shot family keeps pairs (half
    # as many per-tile flags).
    if cta_group is None:
        cta_group = 2 if M > BM and (not ag or (M // world) % (2 * BM) == 0) else 1
        if mode in ("store", "reduce") and N <= 8192 and not (store_all and world > 1):
            cta_group = 1   # (with tiles pushed to peers the pair stays ahead: 380 us against 392 us on 2 GPUs)
        if reduce_scatter and M % (world * 2 * BM) != 0:
            cta_group = 1
    if group_m is None:   # m-tiles per raster group: wider groups pay once a row of tiles no longer fits a wave
        group_m = 16 if N >= 12288 else 8
    if cta_group not in (1, 2):
        raise ValueError("cta_group must be 1 or 2")
    # reduce-scatter: rank r keeps rows [r * M / world, (r + 1) * M / world) of the sum
    rs_rows = 0
    if reduce_scatter:
        if mode != "one_shot":
            raise ValueError("reduce_scatter=True goes with mode='one_shot'")
        if M % (world * BM * cta_group) != 0:
            raise ValueError(f"reduce-scatter needs M to be a multiple of world x {BM * cta_group}")
        rs_rows = M // world
        push, ksplit = True, 1
        mt = rs_rows // (BM * cta_group)     # m-tiles per rank: the raster groups must not straddle ranks
        group_m = max(g for g in range(1, max(1, int(group_m)) + 1) if mt % g == 0)
    ctas = int(ctas_per_rank) if ctas_per_rank else sms // num_local
    ctas -= ctas % cta_group
    tiles_m, tiles_n = -(-M // (BM * cta_group)), -(-N // bn)
    T = tiles_m * tiles_n
    kblocks = -(-K // sub_cols)
    # ---- schedule: whole tiles round-robin, plus (stream-K) a tail of tiles split by k-blocks ----
    units = max(1, ctas // cta_group)
    if stream_k is None:
        # On where it was measured to pay: kernels that keep or push whole tiles (store / reduce), 16-bit elements,
        # at least one full wave of whole tiles before the split part, a ragged last wave.  One GPU, 8192 x N x 4096:
        # N = 3584: 192 -> 181 us, N = 7168: 380 -> 364 us, N = 14336: 654 -> 650 us.  Off where every tile would be
        # split (fewer than two waves of tiles: 1024 x 8192 x 8192 loses 10 - 60 %) and for the summing kernels (not
        # measured).
        # The environment variable IRIS_STREAM_K overrides this default for A/B runs of whole programs: 0 = never,
        # 1 = wherever the kernel can (also with fewer tiles than units).
        eligible = mode in ("store", "reduce") and es == 2 and not tail_split and (ksplit or 1) == 1
        # a wave of whole tiles stays in front of the split part, and the last wave is at most half full (fuller ones
        # measured neutral: 8192 x 5120 x 4096, 0.65 of a wave: 245 - 249 -> 247 us)
        stream_k = eligible and T >= 2 * units and 0 < T % units <= units // 2
        if stream_k and store_all and world > 1:
            # Tiles pushed to every peer: where the pushes, not the MMAs, set the time, the units' ranges ending together
            # only bunches the last pushes (4 GPUs, 8192 x 3584 x 4096 per rank: 320 -> 332 us with stream-K; 2 GPUs,
            # compute-bound: 393 -> 381 us).  Rough rates: 1.4 PFLOP/s, 700 GB/s out of every GPU.
            stream_k = 2.0 * M * N * K / 1.4e15 > (world - 1) * M * N * es / 700e9
        env = os.environ.get("IRIS_STREAM_K")
        if env == "0":
            stream_k = False
        elif env == "1":
            stream_k = eligible
    dp_tiles, sk_units, sk_tiles = T, 0, 0
    if stream_k and T % units != 0:
        sk_tiles = T % units + (units if T >= units else 0)   # the ragged wave plus one full wave
        sk_tiles = min(sk_tiles, T)
        dp_tiles = T - sk_tiles
        # ranges of at least half a tile: a split tile then meets at most four ranges, the finisher's and SK_SLOTS others
        sk_units = max(1, min(units, 2 * sk_tiles))
    if dp_tiles == 0:
        units = sk_units if sk_units else min(units, max(T, 1 if not ag else 8))
    elif not sk_units:
        units = min(units, max(T, 1 if not ag else 8))
    ctas = max(1, units) * cta_group
    # ---- one-shot for short matrices: partials pushed into every rank's inbox, K cut into pieces ----
    max_units = max(1, (sms // num_local) // cta_group)
    do_push = bool(push) if push is not None else (mode == "one_shot" and M <= 2 * BM)
    if mode != "one_shot":
        do_push = False
    ks = 1
    if do_push:
        if ksplit is None:
            per_w = max(1, 16 // world)            # keep (ranks x pieces) summed per chunk at <= 16
            ksplit = max(1, min(max_units // max(T, 1), per_w, kblocks // 4))
        ks = max(1, int(ksplit))
        if ks > 1:
            dp_tiles, sk_units, sk_tiles = T, 0, 0
            ctas = min(max_units, T * ks) * cta_group
    # ---- atomic all-reduce of a short matrix: the K range of every tile is cut into pieces computed by different
    # CTAs, each of which adds its partial tile straight into the outputs (no slots, no summing pass) ----
    if mode == "reduce" and ksplit is not None and int(ksplit) > 1:
        ks = max(1, min(int(ksplit), kblocks))
        if ks > 1:
            dp_tiles, sk_units, sk_tiles = T, 0, 0
            ctas = min(max_units, T * ks) * cta_group
    pulls = mode in ("one_shot", "two_shot")
    # ---- ragged last wave of a whole-tile schedule: cut its tiles into column pieces (nothing to fix up) ----
    tail_tiles, tsplit = 0, 1
    if tail_split and not pulls and not sk_units and ks == 1:
        max_split = min(int(tail_split) if tail_split > 1 else 2, bn // sub_cols)   # pieces are whole sub-tiles
        while max_split > 1 and ((bn // max_split) // cta_group) % 8:
            max_split //= 2
        tail_tiles, tsplit = tail_split_plan(T, max(1, ctas // cta_group), max_split)
    chunks_per_shard = (M // world) // BM if ag else 0
    tile_flags = T * cta_group if pulls else 0
    sk_flags = sk_tiles * cta_group
    # workspace slots of a split tile: one per unit its k-blocks meet, less the unit that finishes it
    sk_slots = 0
    if sk_units:
        S = sk_tiles * kblocks
        sk_slots = max(sk_unit_of((t + 1) * kblocks - 1, S, sk_units) - sk_unit_of(t * kblocks, S, sk_units)
                       for t in range(sk_tiles))
        sk_slots = max(1, sk_slots)
        if sk_slots > SK_SLOTS:
            raise ValueError("stream-K schedule needs more workspace slots per tile than the kernel addresses")
    nflags = FLAG_HEADER + tile_flags + world * chunks_per_shard + sk_flags
    if pulls:
        # One matrix per rank holds both partial buffers (call parity) and, unless the caller brings its own, the
        # output: [partial 0 | partial 1 | out], each padded to whole 256-row tiles, so that one tensor map per rank
        # serves partial stores, partial loads and output stores.
        rows = rs_rows if rs_rows else M
        mp = -(-rows // (2 * BM)) * (2 * BM)
        slots = world * ks if do_push else 1
        if bcast:
            # push two-shot: the keeper of a row block writes its summed rows into every rank's output, which therefore
            # holds all M rows (world blocks) and has to be the symmetric one
            if not rs_rows or own_out:
                raise ValueError("bcast=True goes with reduce_scatter=True and the op's own output buffer")
            out_rows, out_regions = M, world
        else:
            out_rows, out_regions = rows, (0 if own_out else 1)
        regions = 2 * slots + out_regions
        c_rows, part_row0 = regions * mp, (0, slots * mp)
        out_row0 = -1 if own_out else 2 * slots * mp
    else:
        rows, mp, slots, regions, c_rows, part_row0, out_row0, out_rows = M, 0, 0, 0, 0, (0, 0), -1, M
    return GemmPlan(M=M, N=N, K=K, world=world, num_local=num_local, mode=mode, ag=bool(ag), cta_group=cta_group,
                    group_m=int(group_m), rs_rows=rs_rows, ctas_per_rank=ctas, total_tiles=T, kblocks=kblocks,
                    dp_tiles=dp_tiles, sk_units=sk_units, sk_tiles=sk_tiles, push=do_push, ksplit=ks,
                    store_all=bool(store_all) and world > 1, pulls=pulls, chunks_per_shard=chunks_per_shard,
                    tile_flags=tile_flags, sk_flags=sk_flags, nflags=nflags, rows=rows, slot_rows=mp, slots=slots,
                    regions=regions, c_rows=c_rows, part_row0=part_row0, out_row0=out_row0, out_rows=out_rows,
                    bcast=bool(bcast) and bool(rs_rows), bn=bn,
                    tail_tiles=tail_tiles, tail_split=tsplit, sk_slots=sk_slots)
