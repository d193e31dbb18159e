// gemm_schedule.h — the pure index arithmetic of the fused GEMM's tile schedules, usable on host and device.
// The kernel (gemm_fused.cu) calls these; the same functions are exported through C wrappers
// (iris_sched_* in gemm_fused.cu) so that their invariants can be checked on a machine without a GPU
// (tests/test_schedule_cpu.py): every map is a bijection, work is balanced, a keeper has one sender per step.
#pragma once

#if defined(__CUDACC__)
#define IRIS_SCHED_HD __host__ __device__ __forceinline__
#else
#define IRIS_SCHED_HD inline
#endif

namespace iris {
namespace gemm {

struct TileCoord {
  int m_idx, n_idx;
};

// Grouped raster: consecutive tile ids walk down `group_m` m-tiles before moving to the next n-tile, so
// the CTAs of one wave share A rows and B columns in L2 (the reference's GROUP_SIZE_M swizzle,
// examples/07_gemm_all_scatter/gemm_all_scatter.py:158-163).
IRIS_SCHED_HD TileCoord raster(int tile, int tiles_m, int tiles_n, int group_m) {
  const int per_group = group_m * tiles_n;
  const int g = tile / per_group;
  const int first_m = g * group_m;
  const int rest = tiles_m - first_m;
  const int gsz = rest < group_m ? rest : group_m;
  const int in_g = tile - g * per_group;
  TileCoord c;
  c.m_idx = first_m + in_g % gsz;
  c.n_idx = in_g / gsz;
  return c;
}

// With the all-gather prologue the m-tiles are visited shard by shard starting with the rank's own rows:
// logical shard position sp maps to source rank (rank + sp) % world.
IRIS_SCHED_HD int ag_actual_m(int logical_m, int tiles_per_shard, int rank, int world) {
  const int sp = logical_m / tiles_per_shard;
  const int within = logical_m - sp * tiles_per_shard;
  const int s = (rank + sp) % world;
  return s * tiles_per_shard + within;
}

// Two-shot all-reduce: the rank that sums tile t.  A scheduling unit visits tiles u, u + units, u + 2 units, ...;
// rotating the owner with the visit number gives every unit of every rank the same share of the summing work.
IRIS_SCHED_HD int two_shot_owner(int tile, int units, int world) { return ((tile % units) + (tile / units)) % world; }

// Reduce-scatter: the tiles of keeper b's row block are [b * tiles_per_block, (b + 1) * tiles_per_block) in raster
// order.  Step i of rank `rank` is tile i / world of block (rank + 1 + i) % world: at every step the ranks send to
// `world` different keepers, and tile j of every block has been visited by every rank after (j + 1) * world steps.
IRIS_SCHED_HD int rs_tile_of(int step, int rank, int world, int tiles_per_block) {
  return ((rank + 1 + step) % world) * tiles_per_block + step / world;
}

// One piece of work of a scheduling unit: k-blocks [kb0, kb1) of `tile`.
struct Work {
  int tile, kb0, kb1;
  int piece;  // K-split piece of the tile (0 when tiles are not K-split into slots)
  int sub;    // column piece of a tail tile (0 .. tail_split - 1), 0 for a whole tile
  int nsub;   // number of column pieces this tile is cut into (1: the piece is the whole tile)
};

// How many tiles at the end of the raster are cut into column pieces, and into how many, so that the last, ragged
// wave of a persistent schedule keeps every unit busy: with T tiles on G units the last T % G tiles would occupy
// only that many units for a whole tile time.  Cutting each of them into s column pieces (each piece a narrower MMA
// on the same A rows, nothing to fix up afterwards, unlike a K split) turns the wave into (T % G) * s pieces of
// 1 / s tile time.  s is the largest divisor of `max_split` with (T % G) * s <= G; 1 (no split) when the ragged
// wave is more than half full or there is no full wave before it.
IRIS_SCHED_HD void tail_split_plan(int total_tiles, int units, int max_split, int* tail_tiles, int* split) {
  *tail_tiles = 0;
  *split = 1;
  if (units < 1 || total_tiles <= units) return;
  const int r = total_tiles % units;
  if (r == 0 || 2 * r > units) return;
  int s = 1;
  for (int c = 2; c <= max_split; c *= 2)
    if (max_split % c == 0 && r * c <= units) s = c;
  if (s > 1) {
    *tail_tiles = r;
    *split = s;
  }
}

// Stream-K bookkeeping.  The stream-K iterations [0, S) are cut into U ranges with boundaries floor(S * i / U)
// (WorkIter below); the unit whose range holds iteration x is the largest i with floor(S * i / U) <= x.
IRIS_SCHED_HD int sk_unit_of(long long x, long long S, int U) { return (int)(((x + 1) * U - 1) / S); }
// A split tile is finished by the unit that computes its FIRST k-blocks: that piece is the last item of the unit's
// range, while the tile's other pieces are the first items of the following units' ranges, so they are done (or
// nearly) when the finisher asks for them.  Each of those other pieces is parked in a workspace slot of its own,
// slot = (its unit) - (the finisher's unit) - 1.  kSkSlots bounds the slots a tile may need; the planner keeps the
// ranges at least half a tile long, so a tile meets at most four ranges.
constexpr int kSkSlots = 3;

// Persistent + stream-K schedule.  Tiles [0, dp_tiles) are taken whole, round-robin over the units (the reference's
// `for tile_id in range(pid, total_tiles, NUM_SMS)`, examples/07_gemm_all_scatter/gemm_all_scatter.py:153).  The
// remaining tiles form one long sequence of (tile, k-block) iterations that is cut into `sk_units` equal ranges —
// the stream-K decomposition the reference only sketches (matmul_wrapper.py:73-103 computes its statistics, the
// kernels never use them).  A unit's range may end in the middle of a tile; such a tile is finished by the unit that
// holds its first k-blocks (see sk_unit_of above and the epilogue).  With `ksplit` > 1 every tile is instead cut into `ksplit`
// fixed slices of its k-blocks and the (tile, piece) items go round-robin over the units.
// With `tail_tiles` > 0 (whole-tile schedules only) the last `tail_tiles` tiles are not part of the round-robin: each
// is cut into `tail_split` column pieces and the pieces go round-robin over the units after the whole tiles.
struct WorkIter {
  int G, dp_tiles, kblocks, next_dp, ksplit, items;
  int tail0, tail_split, tail_items, next_tail;
  long long it, end;
  IRIS_SCHED_HD WorkIter(int unit, int G_, int total_tiles, int kblocks_, int dp_tiles_, int sk_units, int ksplit_,
                         int tail_tiles = 0, int tail_split_ = 1)
      : G(G_), dp_tiles(dp_tiles_), kblocks(kblocks_), next_dp(unit), ksplit(ksplit_ > 1 ? ksplit_ : 1),
        items(total_tiles * (ksplit_ > 1 ? ksplit_ : 1)), tail0(total_tiles), tail_split(1), tail_items(0),
        next_tail(unit), it(0), end(0) {
    const long long S = (long long)(total_tiles - dp_tiles_) * kblocks_;
    if (S > 0 && unit < sk_units) {
      it = S * unit / sk_units;
      end = S * (unit + 1) / sk_units;
    }
    if (tail_tiles > 0 && tail_split_ > 1 && ksplit == 1 && dp_tiles_ == total_tiles) {
      tail0 = total_tiles - tail_tiles;
      dp_tiles = tail0;
      tail_split = tail_split_;
      tail_items = tail_tiles * tail_split_;
    }
  }
  IRIS_SCHED_HD bool next(Work& w) {
    w.piece = 0;
    w.sub = 0;
    w.nsub = 1;
    if (ksplit > 1) {
      // K-split into inbox slots: item i = (tile i / ksplit, piece i % ksplit), each a fixed slice of the k-blocks
      if (next_dp >= items) return false;
      w.tile = next_dp / ksplit;
      w.piece = next_dp - w.tile * ksplit;
      w.kb0 = (int)((long long)kblocks * w.piece / ksplit);
      w.kb1 = (int)((long long)kblocks * (w.piece + 1) / ksplit);
      next_dp += G;
      return true;
    }
    if (next_dp < dp_tiles) {
      w.tile = next_dp;
      w.kb0 = 0;
      w.kb1 = kblocks;
      next_dp += G;
      return true;
    }
    if (it < end) {
      const int t = (int)(it / kblocks);
      const int kb0 = (int)(it - (long long)t * kblocks);
      const long long left = end - it;
      const int len = (int)((long long)(kblocks - kb0) < left ? (kblocks - kb0) : left);
      w.tile = dp_tiles + t;
      w.kb0 = kb0;
      w.kb1 = kb0 + len;
      it += len;
      return true;
    }
    if (next_tail < tail_items) {
      w.tile = tail0 + next_tail / tail_split;
      w.sub = next_tail % tail_split;
      w.nsub = tail_split;
      w.kb0 = 0;
      w.kb1 = kblocks;
      next_tail += G;
      return true;
    }
    return false;
  }
};

}  // namespace gemm
}  // namespace iris
