// gemm_fused.cu — persistent, warp-specialised GEMM for sm_100a with the collective fused into it.
//
//   C[M, N] = A[M, K] * B[N, K]^T        (both operands K-contiguous; C has the operands' element type)
//
// Element types (template parameter ET): bf16 and fp16 with fp32 accumulation for every mode; float32 multiplied as
// tf32 and int8 with 32-bit integer accumulation (low 8 bits stored) for the store mode.  A ring stage and an
// epilogue sub-tile row are 128 bytes for every type, so "128 x 64" below reads 128 x 32 for float32 and 128 x 128 for
// int8.  Nothing in the launch arguments changes from call to call (the call number lives in device memory), so a
// launch can be captured into a CUDA graph.
//
// Data path per CTA (one CTA per SM; 128 x 256 output tile per CTA, or 256 x 256 per pair of CTAs):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of the A (128 x 64) and B slices into a shared-memory ring,
//               completion on mbarriers.  Every CTA loads for itself; there is no cluster multicast.
//   warp 1      one thread issues tcgen05.mma (M128 N256 K16 with cta_group::1, M256 N256 K16 with cta_group::2);
//               accumulators live in tensor memory, two of them, so the epilogue of tile i overlaps the main loop
//               of tile i+1.
//   warps 2-5   epilogue: tcgen05.ld -> output type -> swizzled shared memory -> the collective:
//                 store     TMA store of the tile into the C buffer of every rank       (GEMM + all-scatter)
//                 reduce    TMA reduce-add of the tile into the C buffer of every rank  (GEMM + atomic all-reduce)
//                 one-shot  tile -> partial buffer (own, or pushed into an inbox slot of every rank) + per-tile flag
//                 two-shot  tile -> own partial buffer + flag on the rank that owns the tile
//   warps 6-9   (one-/two-shot kernels) reducer: waits for a tile's flag, fetches the partials of all ranks (TMA
//               loads into a ring of pull buffers, or plain loads from the local inbox, or NVLS multimem.ld_reduce),
//               adds in fp32 and writes the result to this rank (one-shot) or to every rank (two-shot), while the
//               other warps keep computing.
//   warps 6-7   (other kernels) all-gather prologue: push this rank's rows of A to every peer in slices, each
//               followed by a release increment of the peer's chunk flag; the producer warp waits for a chunk's
//               flag before it loads rows that came from a peer (data is read from LOCAL memory).
//
// What it replaces in the reference: the persistent Triton kernels
// examples/07_gemm_all_scatter/gemm_all_scatter.py:97-255,
// examples/08_gemm_atomics_all_reduce/gemm_atomics_all_reduce.py:94-252 and
// examples/09_gemm_one_shot_all_reduce/gemm_one_shot_all_reduce.py:94-275.
//
// Every wait (mbarrier, flag) is bounded by timeout_ns; on expiry the CTA records a status, raises its
// abort word, lets every role leave its loop, frees its tensor memory and returns.
//
// Several ranks can be simulated by ONE launch on one GPU (num_local > 1, cooperative launch): CTA b works
// as rank rank0 + b / ctas_per_rank.  That is how the multi-rank protocols are tested on a single GPU.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <string.h>

#include <atomic>
#include <mutex>
#include <new>

#include "gemm_fused.cuh"
#include "gemm_schedule.h"
#include "iris/iris.cuh"
#include "iris/nvls.cuh"
#include "iris/ptx_sm100.cuh"

namespace iris {
namespace gemm {

using namespace iris::ptx;

// Sites reported in StatusBlock::where.
enum Site : uint32_t {
  kSiteProducerEmpty = 10,
  kSiteProducerAgFlag = 11,
  kSiteAgEntry = 12,
  kSiteZero = 13,
  kSiteMmaAccEmpty = 20,
  kSiteMmaFull = 21,
  kSiteEpiAccFull = 30,
  kSiteEpiEntry = 31,
  kSiteEpiTileFlag = 32,
  kSitePullFull = 33,
  kSiteEpiStreamK = 34,   // finisher of a split tile waiting for the other pieces (or a schedule out of bounds)
  kSiteDone = 40,
};

__device__ __forceinline__ uint32_t* flag_ptr(const FusedGemmParams& p, int rank, int index) {
  return reinterpret_cast<uint32_t*>(p.heap_base[rank] + p.flags_off) + index;
}
__device__ __forceinline__ StatusBlock* status_ptr(const FusedGemmParams& p, int rank) {
  return reinterpret_cast<StatusBlock*>(p.heap_base[rank] + p.status_off);
}

// Per-tile timestamps (the reference's Timestamps arrays, examples/common/utils.py:45-128, filled with
// atomic_min / atomic_max of s_memrealtime; here one thread per role writes its own slot).
__device__ __forceinline__ void trace(const FusedGemmParams& p, int rank, int record, int slot) {
  if (p.trace_off) {
    uint64_t* t = reinterpret_cast<uint64_t*>(p.heap_base[rank] + p.trace_off);
    t[(size_t)record * kTrSlots + slot] = timer_ns();
  }
}

// Two fp32 values -> one 32-bit word of the output type (round to nearest even).
__device__ __forceinline__ uint32_t pack2(float lo, float hi, bool f16) {
  if (f16) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
// acc[0..8) += the eight 16-bit values of v (bf16 or fp16), in fp32.
__device__ __forceinline__ void acc_x8(float* acc, uint4 v, bool f16) {
  if (f16) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
    return;
  }
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    acc[2 * i] += f.x;
    acc[2 * i + 1] += f.y;
  }
}

// Reduce-scatter reducer, one 128 x 256 part: sums `ns` inbox slots (local memory, `slot_rows` rows apart, first row
// `part_row0`) over rows [mo, mo + 128) and columns [n0, n0 + 256) and writes the bf16 rows to `outp` (row pitch
// `out_pitch` bytes).  Called by the 128 reducer threads (`rt` = 0..127).  A warp reads whole 512-byte rows (one
// 16-byte load per lane), four rows of four slots in flight per thread.  Kept out of line so that its registers do
// not add to those of the kernel's other roles.
// With `bcast` (push two-shot all-reduce) every summed row is written to the outputs of all `W` ranks instead: `outp`
// is then the offset of the output from the heap base and the row index is the global one (`mo + out_row_add`); on a
// heap bound to an NVLS multicast object (`mc` != 0) that is one multimem.st per 16 bytes.
// Few arguments on purpose (everything else is read from the launch parameters): the call sits in a role whose
// registers are already scarce.
__device__ __noinline__ void rs_sum_part(const FusedGemmParams& p, int rank, int ns, int mo, int n0, int rt, bool f16,
                                         int part_row0) {
  constexpr int kSlotsInFlight = 4;
  const int W = p.world, N = p.N, bn = p.bn, slot_rows = p.part_slot_rows;
  const bool bcast = p.rs_bcast != 0;
  const int out_row_add = bcast ? rank * p.rs_rows : 0;
  const uint64_t mc = bcast ? p.mc_base : 0;
  const uint64_t* heap_base = p.heap_base;
  const uint8_t* inbox = reinterpret_cast<const uint8_t*>(p.heap_base[rank] + p.partial_off);
  // plain reduce-scatter: address of the kept block; broadcast: offset of the output from the heap base
  uint8_t* outp = bcast ? reinterpret_cast<uint8_t*>(p.partial_off + (uint64_t)p.out_row0 * p.N * 2)
                  : p.out_row0 >= 0
                      ? reinterpret_cast<uint8_t*>(p.heap_base[rank] + p.partial_off) + (uint64_t)p.out_row0 * p.N * 2
                      : reinterpret_cast<uint8_t*>(p.heap_base[rank] + p.out_off);
  const uint64_t out_pitch = (bcast || p.out_row0 >= 0) ? (uint64_t)p.N * 2 : (uint64_t)p.ldo * 2;
  const int rw = rt >> 5, rl = rt & 31;
  const int col = n0 + rl * 8;
  if (col >= N || rl * 8 >= bn) return;  // past the matrix edge / past this (narrower) tile
  const uint64_t row_bytes = (uint64_t)N * 2;
  const uint64_t slot_bytes = (uint64_t)slot_rows * row_bytes;
#pragma unroll 1
  for (int r0 = rw * 32; r0 < rw * 32 + 32; r0 += 4) {
    float a4[4][8];
#pragma unroll
    for (int u = 0; u < 4; ++u)
#pragma unroll
      for (int j = 0; j < 8; ++j) a4[u][j] = 0.f;
    const uint8_t* src = inbox + (uint64_t)(part_row0 + mo + r0) * row_bytes + (uint64_t)col * 2;
#pragma unroll 1
    for (int sl = 0; sl < ns; sl += kSlotsInFlight) {
      // [slot][row]: sixteen 16-byte loads in flight per thread, 32 KB per CTA: the loop is bound by the latency of
      // local memory under load, and with 8 ranks a part is 512 KB
      uint4 v[kSlotsInFlight][4];
#pragma unroll
      for (int q = 0; q < kSlotsInFlight; ++q) {
        if (sl + q < ns) {
#pragma unroll
          for (int u = 0; u < 4; ++u)
            v[q][u] = ld_v4_stream(reinterpret_cast<const uint4*>(src + (sl + q) * slot_bytes + u * row_bytes));
        }
      }
#pragma unroll
      for (int q = 0; q < kSlotsInFlight; ++q) {
        if (sl + q < ns) {
#pragma unroll
          for (int u = 0; u < 4; ++u) acc_x8(a4[u], v[q][u], f16);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      uint4 o;
      o.x = pack2(a4[u][0], a4[u][1], f16);
      o.y = pack2(a4[u][2], a4[u][3], f16);
      o.z = pack2(a4[u][4], a4[u][5], f16);
      o.w = pack2(a4[u][6], a4[u][7], f16);
      if (!bcast) {
        st_v4(reinterpret_cast<uint4*>(outp + (uint64_t)(mo + r0 + u) * out_pitch + (uint64_t)col * 2), o);
      } else {
        const uint64_t off = reinterpret_cast<uint64_t>(outp) + (uint64_t)(mo + out_row_add + r0 + u) * out_pitch +
                             (uint64_t)col * 2;
        if (mc) {
          nvls::st_v4(reinterpret_cast<void*>(mc + off), o);
        } else {
          for (int q = 0; q < W; ++q) st_v4(reinterpret_cast<uint4*>(heap_base[(rank + 1 + q) % W] + off), o);
        }
      }
    }
  }
}

__device__ __forceinline__ void red_relaxed_gpu_add(uint32_t* p, uint32_t v) {
  asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void red_add_v4_f32_gpu(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.gpu.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}

// Per-CTA-group configuration.  CG = 1: one CTA per 128 x 256 tile.  CG = 2: a pair of CTAs (one cluster on the
// two SMs of a TPC) per 256 x 256 tile; each CTA loads its own 128 rows of A and its own 128 of the 256 B rows,
// one thread of the leader CTA issues cta_group::2 MMAs that read both CTAs' shared memory, and each CTA ends up
// with its 128 x 256 half of the accumulator in its own tensor memory.  Loads stay per-CTA (no multicast).
// PULL (one-/two-shot all-reduce): the main ring gives up stages for a ring of 16 KB "pull" buffers into which
// the partial sub-tiles of all ranks are fetched with TMA loads (a peer's memory included, no multicast).
template <int CG, bool PULL>
struct Cfg {
  static constexpr int kStages = CG == 1 ? (PULL ? 3 : 4) : (PULL ? 4 : 6);
  static constexpr int kBRows = BN / CG;
  static constexpr int kBStage = kBRows * BK * 2;
  static constexpr int kStage = kAStageBytes + kBStage;
  static constexpr int kPullBufs = PULL ? (CG == 1 ? 2 : 3) : 0;  // ring of fetched partial sub-tiles
  static constexpr int kRedOutBufs = PULL ? 1 : 0;                // reducer's staging buffer for result stores
  static constexpr int kTilesBytes =
      kStages * kStage + (kEpiBufs + kPullBufs + kRedOutBufs) * kEpiStageBytes;
  static_assert(kTilesBytes <= kSmemTiles, "shared-memory budget");
};

template <int CG, bool PULL, int ET>
__global__ void __launch_bounds__(PULL ? kThreadsPull : kThreads, 1)
    fused_gemm_kernel(const __grid_constant__ FusedGemmParams p) {
  using C = Cfg<CG, PULL>;
  constexpr int kStages = C::kStages;
  extern __shared__ uint8_t smem_raw[];
  // 128-byte-swizzled tiles need 1024-byte alignment (identical offsets in both CTAs of a pair).
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t smem_base = smem_u32(smem);
  const uint32_t epi_base = smem_base + kStages * C::kStage;
  const uint32_t pull_base = epi_base + kEpiBufs * kEpiStageBytes;
  const uint32_t redout_base = pull_base + C::kPullBufs * kEpiStageBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
  const uint32_t bar_base = smem_u32(bars);
  // barrier slots: full[6], empty[6], acc_full[2], acc_empty[2], pull_full[4]
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (6 + s); };
  auto acc_full_bar = [&](int b) { return bar_base + 8u * (12 + b); };
  auto acc_empty_bar = [&](int b) { return bar_base + 8u * (14 + b); };
  auto pull_full_bar = [&](int b) { return bar_base + 8u * (16 + b); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 20);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile uint32_t* epi_ok = tmem_slot + 2;
  volatile uint32_t* red_ok = tmem_slot + 3;
  volatile uint32_t* ag_ok = tmem_slot + 4;
  volatile uint32_t* never = tmem_slot + 5;  // stays 0: "abort" word for waits that must not be cut short
  // this call, derived from the call counter in device memory: [0] call number = value of the entry flags, [1] value
  // the per-tile / per-chunk flags reach, [2] value the arrival counter reaches, [3] first row of the partial buffer
  volatile uint32_t* callv = tmem_slot + 6;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int lr = blockIdx.x / p.ctas_per_rank;   // local rank index
  const int cta = blockIdx.x - lr * p.ctas_per_rank;
  const int pr = (CG == 2) ? (int)cluster_ctarank() : 0;  // position in the CTA pair; 0 = leader
  const bool leader = pr == 0;
  const int unit = cta / CG;                      // tile-scheduling unit (CTA or CTA pair) within the rank
  const int G = p.ctas_per_rank / CG;
  const int rank = p.rank0 + lr;
  const int W = p.world;
  StatusBlock* status = status_ptr(p, rank);

  constexpr int TM = BM * CG;                     // rows of a scheduling unit's tile
  const int tiles_m = (p.M + TM - 1) / TM;
  const int bn = p.bn;                            // tile width of this launch (64, 128 or 256)
  constexpr bool f16 = ET == kFp16;               // which 16-bit type, where the code below handles 16-bit values
  constexpr int ES = elem_size(ET);               // bytes per element of A, B and C
  constexpr int BKE = 128 / ES;                   // K elements per ring stage: one 128-byte swizzle row
  constexpr int EC = 128 / ES;                    // output columns per epilogue sub-tile: 128-byte rows again
  static_assert(!PULL || ES == 2, "the summing kernels exist for the 16-bit types only");
  const int tiles_n = (p.N + bn - 1) / bn;
  const int total_tiles = tiles_m * tiles_n;
  const int kblocks = (p.K + BKE - 1) / BKE;
  const int tiles_per_shard = p.ag ? (p.M / W) / TM : 0;
  const int chunks_per_shard = p.ag ? (p.M / W) / BM : 0;  // all-gather flags are per 128 rows
  // Two-shot: the rank that sums tile t.  A scheduling unit visits tiles u, u + G, u + 2G, ...; rotating the owner
  // with the visit number gives every unit of every rank the same share of the summing work.
  auto owner_of = [&](int t) { return two_shot_owner(t, G, W); };
  // Reduce-scatter: the tiles of one keeper's row block are contiguous in raster order (the host picks group_m so):
  // block b is [b * rs_tpc, (b + 1) * rs_tpc).  Step i of a rank's schedule is tile i / W of block (rank + 1 + i) % W:
  // at every step the W ranks send to W different keepers, the link is used evenly from the first tile to the last,
  // and tile j of every block is complete on its keeper after about (j + 1) * W steps, so that the keepers' reducer
  // warps sum while the tensor cores are still busy with later tiles.
  const int rs_tpc = p.rs_rows > 0 ? (p.rs_rows / TM) * tiles_n : 0;  // tiles per row block
  auto tile_of = [&](int i) { return p.rs_rows > 0 ? rs_tile_of(i, rank, W, rs_tpc) : i; };

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      mbar_init(full_bar(s), 1);
      mbar_init(empty_bar(s), 1);
    }
    for (int b = 0; b < kAccBufs; ++b) {
      mbar_init(acc_full_bar(b), 1);
      mbar_init(acc_empty_bar(b), 4 * CG);  // one arrival per epilogue warp of every CTA of the group
    }
    for (int b = 0; b < C::kPullBufs; ++b) mbar_init(pull_full_bar(b), 1);
    *abort_flag = 0;
    *epi_ok = 1;
    *red_ok = 1;
    *ag_ok = 1;
    *never = 0;
    {
      const int my_rank = p.rank0 + blockIdx.x / p.ctas_per_rank;
      const uint32_t call = *reinterpret_cast<volatile uint32_t*>(flag_ptr(p, my_rank, 2)) + 1u;
      callv[0] = call;
      callv[1] = p.per_flag * call;
      callv[2] = call * (uint32_t)p.world * (uint32_t)p.ctas_per_rank;
      callv[3] = (uint32_t)((call & 1u) ? p.part_row0_odd : p.part_row0);
    }
    mbar_fence_init();
    prefetch_tensormap(&p.tmA[lr]);
    prefetch_tensormap(&p.tmB[lr]);
  }
  if (warp == 1) {
    if (CG == 1) {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
      tmem_relinquish();
    } else {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);
      tmem_relinquish_pair();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (CG == 2) cluster_sync_all();  // the partner's barriers exist before anything arrives on them
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  // trace: when this CTA was ready to work / left (slots of the record of the first tile it handles)
  if (p.trace_off && threadIdx.x == 0 && unit < total_tiles) trace(p, rank, tile_of(unit) * CG + pr, kTrCtaBegin);

  // Entry flag: tell every rank that this rank has started call `epoch` (its output buffers are ready to be
  // written by peers).  One thread of one CTA per rank.
  // The flag orders nothing written by this kernel (it has written nothing yet); what a peer relies on, the end of
  // this rank's previous call, is ordered by the kernel boundary.  One fence, then relaxed stores: a release store
  // per peer would wait for the previous peer's acknowledgement each time, a link round trip per rank.
  if (p.zero_bytes) {
    // Atomic all-reduce of a short matrix: the output, which every rank adds into, is cleared here instead of by a
    // launch of its own.  Every CTA clears its share, counts itself on a local counter, and the entry flags (which
    // tell the peers that this rank's output may be added into) go out only when all CTAs of the rank have done so.
    uint8_t* outp = reinterpret_cast<uint8_t*>(p.heap_base[rank] + p.c_off);
    const uint64_t n16 = p.zero_bytes / 16;
    for (uint64_t i = (uint64_t)cta * blockDim.x + threadIdx.x; i < n16; i += (uint64_t)p.ctas_per_rank * blockDim.x)
      st_v4(reinterpret_cast<uint4*>(outp) + i, make_uint4(0u, 0u, 0u, 0u));
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
      red_relaxed_gpu_add(flag_ptr(p, rank, 1), 1u);
      if (cta == 0 &&
          wait_until_ge(flag_ptr(p, rank, 1), callv[0] * (uint32_t)p.ctas_per_rank, p.timeout_ns, status, kSiteZero, rank,
                        0) != kOk)
        *abort_flag = 1;
    }
  }
  if (W > 1 && cta == 0 && threadIdx.x == 0) {
    fence_sys();
    for (int i = 0; i < W; ++i) {
      const int t = (rank + 1 + i) % W;
      st_relaxed_sys(flag_ptr(p, t, 8 + rank), callv[0]);
    }
  }

  if (warp == 0) {
    // ------------------------------------------------------------------------------------------
    // TMA producer (every CTA loads its own A rows and its own share of the B rows)
    // ------------------------------------------------------------------------------------------
    if (lane == 0) {
      int stage = 0;
      uint32_t phase = 0;
      uint32_t fills = 0;  // ring slots filled so far
      bool ok = true;
      WorkIter sched(unit, G, total_tiles, kblocks, p.dp_tiles, p.sk_units, p.ksplit, p.tail_tiles, p.tail_split);
      Work w;
      while (ok && sched.next(w)) {
        const int tile = tile_of(w.tile);
        TileCoord tc = raster(tile, tiles_m, tiles_n, p.group_m);
        if (p.ag) tc.m_idx = ag_actual_m(tc.m_idx, tiles_per_shard, rank, W);
        const int row0 = tc.m_idx * TM + pr * BM;
        // Columns of this piece of work: the whole tile, or one of the column pieces of a tail tile.
        const int wn = bn / w.nsub;                         // width of the piece
        const int col0 = tc.n_idx * bn + w.sub * wn;        // its first column = first row of B^T
        const int b_rows = wn / CG;                         // rows of B^T this CTA loads per k-block
        const uint32_t stage_tx = (uint32_t)(kAStageBytes + b_rows * 128);  // 128-byte rows of K, whatever the type
        if (p.ag && row0 < p.M) {
          const int Ms = p.M / W;
          const int src = row0 / Ms;
          if (src != rank) {
            const int chunk = (row0 - src * Ms) / BM;
            const uint32_t* f = flag_ptr(p, rank, p.ag_flag_base + src * chunks_per_shard + chunk);
            if (wait_until_ge(f, callv[1], p.timeout_ns, status, kSiteProducerAgFlag, rank, tile) != kOk) {
              *abort_flag = 1;
              ok = false;
              break;
            }
            fence_proxy_async_all();  // peer wrote with ordinary stores; TMA reads through the async proxy
          }
        }
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1, p.timeout_ns, abort_flag)) {
            record_status(status, kTimeout, kSiteProducerEmpty, rank, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * C::kStage;
          const uint32_t b_dst = a_dst + kAStageBytes;
          // B^T rows of a whole tile come through tmB (box of bn / CG rows), those of a column piece of a tail tile
          // through tmBt (a box as tall as the piece needs): one load either way.
          const CUtensorMap* tm_b = w.nsub > 1 ? &p.tmBt[lr] : &p.tmB[lr];
          if (CG == 1) {
            mbar_expect_tx(full_bar(stage), stage_tx);
            tma_load_2d(a_dst, &p.tmA[lr], kb * BKE, row0, full_bar(stage));
            tma_load_2d(b_dst, tm_b, kb * BKE, col0, full_bar(stage));
          } else {
            // Both CTAs' bytes are counted on the leader's barrier, which the leader arms for the pair.
            const uint32_t lead_full = mapa_shared(full_bar(stage), 0);
            if (leader) mbar_expect_tx(full_bar(stage), 2 * stage_tx);
            tma_load_2d_pair(a_dst, &p.tmA[lr], kb * BKE, row0, lead_full);
            tma_load_2d_pair(b_dst, tm_b, kb * BKE, col0 + pr * b_rows, lead_full);
          }
          ++fills;
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
      }
      if ((!ok || *abort_flag) && leader) {
        // Leaving early: loads already issued still write into this CTA's (and, for a pair, the partner's) shared
        // memory.  Wait, bounded, for the last fill of every ring slot; the pair's barriers live in the leader and
        // count both CTAs' bytes, and the partner stays until the cluster barrier of the teardown.
        for (int s2 = 0; s2 < kStages; ++s2) {
          const uint32_t n = (fills + kStages - 1 - s2) / kStages;  // fills of slot s2
          if (n > 0) mbar_wait(full_bar(s2), (n - 1) & 1, 200000, never);
        }
      }
    }
  } else if (warp == 1) {
    // ------------------------------------------------------------------------------------------
    // MMA issuer (one thread; with CTA pairs only the leader's)
    // ------------------------------------------------------------------------------------------
    if (lane == 0 && leader) {
      // instruction descriptors per piece width (bn, and bn / tail_split for the column pieces of tail tiles)
      auto idesc_for = [](int n) {
        return ET == kTf32 ? umma_idesc_tf32(TM, n) : ET == kInt8 ? umma_idesc_s8(TM, n) : umma_idesc_f16(TM, n, !f16);
      };
      const uint32_t idesc_tile = idesc_for(bn);
      const uint32_t idesc_tail = idesc_for(bn / (p.tail_split > 1 ? p.tail_split : 1));
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      WorkIter sched(unit, G, total_tiles, kblocks, p.dp_tiles, p.sk_units, p.ksplit, p.tail_tiles, p.tail_split);
      Work w;
      while (ok && sched.next(w)) {
        const int tile = tile_of(w.tile);
        if (!mbar_wait(acc_empty_bar(acc), acc_phase ^ 1, p.timeout_ns, abort_flag)) {
          record_status(status, kTimeout, kSiteMmaAccEmpty, rank, tile, acc);
          *abort_flag = 1;
          break;
        }
        tc_fence_after();
        trace(p, rank, tile * CG, kTrMmaBegin);
        const uint32_t d_tmem = tmem_base + acc * BN;
        const uint32_t idesc = w.nsub > 1 ? idesc_tail : idesc_tile;
        for (int kb = w.kb0; kb < w.kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase, p.timeout_ns, abort_flag)) {
            record_status(status, kTimeout, kSiteMmaFull, rank, tile, kb);
            *abort_flag = 1;
            ok = false;
            break;
          }
          tc_fence_after();
          const uint32_t a_addr = smem_base + stage * C::kStage;
          const uint32_t b_addr = a_addr + kAStageBytes;
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k) {
            const uint64_t a_desc = umma_desc_k_sw128(a_addr + k * UMMA_K * 2);
            const uint64_t b_desc = umma_desc_k_sw128(b_addr + k * UMMA_K * 2);
            const uint32_t accumulate = (kb > w.kb0 || k > 0) ? 1u : 0u;  // the first MMA of a piece overwrites
            // every kind covers 32 bytes of K per instruction: 16 16-bit, 8 tf32 or 32 8-bit elements
            if constexpr (ET == kTf32) {
              if (CG == 1) umma_tf32_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
              else umma_tf32_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
            } else if constexpr (ET == kInt8) {
              if (CG == 1) umma_i8_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
              else umma_i8_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
            } else {
              if (CG == 1) umma_f16_ss(d_tmem, a_desc, b_desc, idesc, accumulate);
              else umma_f16_ss_pair(d_tmem, a_desc, b_desc, idesc, accumulate);
            }
          }
          // Free the ring slot (in both CTAs of a pair) once these MMAs have read it.
          if (CG == 1) {
            umma_commit(empty_bar(stage));
          } else {
            umma_commit_pair(mapa_shared(empty_bar(stage), 0));
            umma_commit_pair(mapa_shared(empty_bar(stage), 1));
          }
          if (++stage == kStages) {
            stage = 0;
            phase ^= 1;
          }
        }
        if (!ok) break;
        trace(p, rank, tile * CG, kTrMmaEnd);  // issue time of the last MMA, not its completion
        if (CG == 1) {
          umma_commit(acc_full_bar(acc));  // accumulator complete
        } else {
          umma_commit_pair(mapa_shared(acc_full_bar(acc), 0));
          umma_commit_pair(mapa_shared(acc_full_bar(acc), 1));
        }
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1;
        }
      }
    }
  } else if (warp < 6) {
    // ------------------------------------------------------------------------------------------
    // Epilogue (128 threads): this CTA's 128 x 256 part of the tile
    // ------------------------------------------------------------------------------------------
    const int et = threadIdx.x - 64;
    const bool issuer = (et == 0);
    const int quad = warp & 3;          // tensor-memory lane quadrant this warp may read
    const int row = quad * 32 + lane;   // row of the tile held by this thread
    const bool pulls = (p.mode == kEpiOneShot || p.mode == kEpiTwoShot);
    const bool push_all =
        ((p.mode == kEpiStore || p.mode == kEpiReduce) && p.store_all && W > 1) || (pulls && p.push_partials && W > 1);
    // Nothing of this call is pushed or published before every peer has entered the call (finished the previous one).
    // For pushes into a peer's output that keeps the previous result intact until the peer is done with it.  For the
    // one-/two-shot and reduce-scatter partials (whose buffers alternate by call parity) it keeps the per-tile flags
    // exact: they are cumulative counters over all sources, and a rank one call ahead could otherwise raise a flag to
    // this call's target while a slow rank's partial of this call is still missing.  The entry flags are written at
    // kernel start and the first publish comes a whole main loop later, so the wait is normally already satisfied.
    // Two-shot result pushes are made (and guarded the same way) by the reducer warps.
    const bool need_entry = W > 1 && (push_all || pulls);
    // How finished sub-tiles leave (GEMM + all-scatter only; every other mode has one issuing thread and TMA):
    const int push_kind =
        (!PULL && (p.mode == kEpiStore || p.mode == kEpiReduce) && push_all) ? p.push_kind : (int)kPushTma;
    const bool direct = push_kind >= kPushStores;                 // the 128 threads copy the staged sub-tile themselves
    const int nlead = push_kind == kPushTmaSpread ? 4 : 1;        // threads that issue TMA stores (lane 0 of a warp)
    const int lead_idx = warp - 2;
    const bool lead = lane == 0 && lead_idx < nlead;              // lead 0 is `issuer`
    int acc = 0;
    uint32_t acc_phase = 0;
    int ebuf = 0;
    const uint64_t evict_first = l2_policy_evict_first();
    int pending_tile = -1;  // one-/two-shot: tile whose partial is stored but not yet published
    const bool publish_early = pulls && p.push_partials && W > 1;
    bool entered = !need_entry;

    // Make a stored partial tile known: one release fence, then a relaxed increment of the tile's flag on every rank
    // (two-shot: only on the rank that sums the tile).  Called by the issuer after the tile's stores completed.
    auto publish_tile = [&](int t) {
      fence_proxy_async_all();
      fence_sys();
      for (int i = 0; i < W; ++i) {
        const int dst = (rank + 1 + i) % W;
        if (p.mode == kEpiTwoShot && dst != owner_of(t)) continue;
        if (p.rs_rows > 0 && dst != t / rs_tpc) continue;  // reduce-scatter: only the keeper of the rows sums them
        red_relaxed_sys_add(flag_ptr(p, dst, p.tile_flag_base + t * CG + pr), 1u);
      }
    };
    bool ok_all = true;
    WorkIter sched(unit, G, total_tiles, kblocks, p.dp_tiles, p.sk_units, p.ksplit, p.tail_tiles, p.tail_split);
    Work w;
    while (sched.next(w)) {
      const int tile = tile_of(w.tile);
      TileCoord tc = raster(tile, tiles_m, tiles_n, p.group_m);
      if (p.ag) tc.m_idx = ag_actual_m(tc.m_idx, tiles_per_shard, rank, W);
      // Stream-K: a piece that covers only part of the tile's k-blocks.  The piece with the tile's first k-blocks (the
      // last item of its unit's range) finishes the tile: it adds the other pieces, which their units parked as fp32 in
      // workspace slots and counted on the tile's counter, to its own accumulator on the way out of tensor memory.
      const bool whole = (w.kb0 == 0 && w.kb1 == kblocks) || p.ksplit > 1;  // a K-split piece is a slot of its own
      int sk_add = 0;               // finisher: pieces to add from the workspace
      int sk_slot = -1;             // other pieces: the slot to park the accumulator in
      float4* sk_ws = nullptr;      // workspace of this CTA's part of the tile: [slot][group of 4 columns][row]
      uint32_t* sk_cnt = nullptr;   // pieces of the tile parked so far
      if (!whole) {
        const int t_sk = tile - p.dp_tiles;
        const long long S = (long long)(total_tiles - p.dp_tiles) * kblocks;
        const int head = sk_unit_of((long long)t_sk * kblocks, S, p.sk_units);
        const size_t part = (size_t)t_sk * CG + pr;
        sk_ws = reinterpret_cast<float4*>(p.heap_base[rank] + p.ws_off) + part * p.sk_slots * (size_t)(BM * BN / 4);
        sk_cnt = flag_ptr(p, rank, p.sk_flag_base + (int)part);
        if (w.kb0 > 0) sk_slot = unit - head - 1;
        else sk_add = sk_unit_of((long long)(t_sk + 1) * kblocks - 1, S, p.sk_units) - head;
      }
      // Partials pushed into a peer's inbox: the previous tile is published here, before this tile's stores exist, so
      // that the system-scope fence of the publish has no younger stores of this thread behind it (reduce-scatter on 4
      // GPUs: 283 -> 278 us against publishing after the next tile's stores were issued).
      if (publish_early && issuer && pending_tile >= 0) {
        bulk_wait<0>();
        publish_tile(pending_tile);
        pending_tile = -1;
      }
      // Uniform decision for the whole epilogue group: one thread waits, everybody reads the verdict.
      if (issuer) {
        bool ok = mbar_wait(acc_full_bar(acc), acc_phase, p.timeout_ns, abort_flag);
        if (!ok) record_status(status, kTimeout, kSiteEpiAccFull, rank, tile, acc);
        if (ok && !whole && (sk_slot >= p.sk_slots || sk_add > p.sk_slots || (sk_slot < 0 && sk_add < 1))) {
          record_status(status, kTimeout, kSiteEpiStreamK, rank, tile, sk_slot);  // a schedule the planner must not make
          ok = false;
        }
        if (ok && sk_add > 0) {
          // the other pieces were first in their units' ranges: normally this is already satisfied
          ok = wait_until_ge(sk_cnt, (uint32_t)sk_add, p.timeout_ns, status, kSiteEpiStreamK, rank, tile) == kOk;
          if (ok) *reinterpret_cast<volatile uint32_t*>(sk_cnt) = 0u;  // ready for the next call
        }
        if (ok && !entered) {
          // Before the first push of this call: every peer must have entered the call.
          for (int i = 0; i < W && ok; ++i) {
            const int t = (rank + 1 + i) % W;
            ok = wait_until_ge(flag_ptr(p, rank, 8 + t), callv[0], p.timeout_ns, status, kSiteEpiEntry, rank, t) == kOk;
          }
        }
        *epi_ok = ok ? 1u : 0u;
      }
      named_barrier_sync(1, 128);
      const bool ok = *epi_ok != 0;
      named_barrier_sync(1, 128);
      if (!ok) {
        ok_all = false;
        break;
      }
      entered = true;
      tc_fence_after();
      if (issuer) trace(p, rank, tile * CG + pr, kTrEpiBegin);

      const int wn = bn / w.nsub;                    // width of this piece: the tile, or a column piece of a tail tile
      const int ncol0 = tc.n_idx * bn + w.sub * wn;  // its first column inside this rank's N
      const int nchunks = wn / EC;
      const int x_base = (pulls ? 0 : rank * p.col_off_per_rank) + ncol0;
      const int y = tc.m_idx * TM + pr * BM;
      // row inside the tmC matrix: partial buffer of this call's parity, inbox slot of (rank, piece) when pushing
      const int slot = p.push_partials ? rank * (p.ksplit > 1 ? p.ksplit : 1) + w.piece : 0;
      const int keeper = p.rs_rows > 0 ? tile / rs_tpc : -1;  // reduce-scatter: the rank that keeps these rows
      const int y_st = (pulls ? (int)callv[3] + slot * p.part_slot_rows : 0) + y - (keeper > 0 ? keeper * p.rs_rows : 0);

      int groups_this_tile = 0;  // bulk groups the issuer committed for this tile
      if (sk_slot >= 0) {
        // Park this piece: 32 columns at a time out of tensor memory, four columns (16 bytes) per store, the 32 rows of
        // a warp next to one another so that every store instruction writes one 512-byte run.
        float4* dst = sk_ws + (size_t)sk_slot * (BM * BN / 4) + row;
#pragma unroll 1
        for (int c = 0; c < bn / 32; ++c) {
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * 32, v);
          tmem_wait_ld();
#pragma unroll
          for (int j = 0; j < 8; ++j)
            __stcg(dst + (size_t)(c * 8 + j) * BM, make_float4(__uint_as_float(v[4 * j]), __uint_as_float(v[4 * j + 1]),
                                                              __uint_as_float(v[4 * j + 2]), __uint_as_float(v[4 * j + 3])));
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CG == 1) mbar_arrive(acc_empty_bar(acc));
          else mbar_arrive_cluster(mapa_shared(acc_empty_bar(acc), 0));
        }
        if (++acc == kAccBufs) {
          acc = 0;
          acc_phase ^= 1;
        }
        __threadfence();  // this thread's stores are visible before the count says so
        named_barrier_sync(1, 128);
        if (issuer) atomic_add<Sem::release, Scope::gpu>(sk_cnt, 1u, 0, 0, p.heap_base);
        continue;  // the unit with the tile's first k-blocks finishes it
      }
#pragma unroll 1
      for (int c = 0; c < nchunks; ++c) {
        const bool live = ncol0 + c * EC < p.N && y < p.M;  // parts past the matrix edge are skipped
        // o[0..32): this thread's 128 bytes of the sub-tile's row, as they go to shared memory
        uint32_t o[32];
        if constexpr (ES != 2) {
          // 32-bit results are the accumulator's bits; 8-bit results are the low byte of each 32-bit sum, four to a word
          const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * EC;
          if constexpr (ET == kTf32) {
            tmem_ld_32x32b_x32(taddr, o);
            tmem_wait_ld();
          } else {
#pragma unroll
            for (int s4 = 0; s4 < 4; ++s4) {
              uint32_t v[32];
              tmem_ld_32x32b_x32(taddr + 32 * s4, v);
              tmem_wait_ld();
#pragma unroll
              for (int j = 0; j < 8; ++j)
                o[8 * s4 + j] = (v[4 * j] & 0xffu) | ((v[4 * j + 1] & 0xffu) << 8) | ((v[4 * j + 2] & 0xffu) << 16) |
                                (v[4 * j + 3] << 24);
            }
          }
        } else {
          uint32_t v[kEpiCols];
          const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + acc * BN + c * kEpiCols;
          tmem_ld_32x32b_x32(taddr, v);
          tmem_ld_32x32b_x32(taddr + 32, v + 32);
          tmem_wait_ld();
#pragma unroll 1
          for (int s2 = 0; s2 < sk_add; ++s2) {
            // finishing a split tile: add the pieces the other units parked (L2 reads, never through L1)
            const float4* src = sk_ws + (size_t)s2 * (BM * BN / 4) + (size_t)(c * (kEpiCols / 4)) * BM + row;
#pragma unroll
            for (int j = 0; j < kEpiCols / 4; ++j) {
              const float4 f = __ldcg(src + (size_t)j * BM);
              v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + f.x);
              v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + f.y);
              v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + f.z);
              v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + f.w);
            }
          }
#pragma unroll
          for (int j = 0; j < 32; ++j) o[j] = pack2(__uint_as_float(v[2 * j]), __uint_as_float(v[2 * j + 1]), f16);
        }
        if (c == nchunks - 1) {
          // The accumulator has been read completely: hand it back to the MMA warp (of the leader CTA).
          tc_fence_before();
          __syncwarp();
          if (lane == 0) {
            if (CG == 1) mbar_arrive(acc_empty_bar(acc));
            else mbar_arrive_cluster(mapa_shared(acc_empty_bar(acc), 0));
          }
        }
        if (!live) continue;  // uniform over the group
        // The staging buffer was last used two sub-tiles ago: its TMA reads must have finished (every issuing thread
        // waits for its own bulk groups; threads that copy the buffer themselves are past it at the barrier).
        if (lead && !direct) bulk_wait_read<kEpiBufs - 1>();
        named_barrier_sync(1, 128);
        const uint32_t sbase = epi_base + ebuf * kEpiStageBytes + row * 128;
#pragma unroll
        for (int j = 0; j < 8; ++j)  // 128-byte swizzle, as the tensor map expects
          st_shared_v4(sbase + ((j ^ (row & 7)) << 4), o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        if (!direct) fence_proxy_async_smem();
        named_barrier_sync(1, 128);
        if (direct) {
          // Copy the staged 128-row sub-tile (128 bytes per row) out with 16-byte stores: 8 lanes cover one 128-byte row
          // segment, a warp four rows.  Element (r, j) of the buffer sits at the swizzled position the staging loop wrote
          // it to.
          const uint32_t src = epi_base + ebuf * kEpiStageBytes;
          const int x = x_base + c * EC;
          uint4 vv[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int idx = i * 128 + et, r = idx >> 3, j = idx & 7;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(vv[i].x), "=r"(vv[i].y), "=r"(vv[i].z), "=r"(vv[i].w)
                         : "r"(src + r * 128 + ((j ^ (r & 7)) << 4)));
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const int idx = i * 128 + et, r = idx >> 3, j = idx & 7;
            if (y + r < p.M) {
              const uint64_t off = p.c_off + ((uint64_t)(y + r) * p.ldc + x) * ES + j * 16;
              if (push_kind == kPushMultimem) {
                // one instruction, delivered (store) or added (reduce) by the switch on every rank's copy
                void* mc = reinterpret_cast<void*>(p.mc_base + off);
                if (ES == 2 && p.mode == kEpiReduce) {
                  if (f16) nvls::red_add_f16x8(mc, vv[i]);
                  else nvls::red_add_bf16x8(mc, vv[i]);
                } else {
                  nvls::st_v4(mc, vv[i]);
                }
              } else {
                for (int q = 0; q < W; ++q)  // peers first, starting with the next rank; own copy last
                  st_v4(reinterpret_cast<uint4*>(p.heap_base[(rank + 1 + q) % W] + off), vv[i]);
              }
            }
          }
        } else if (lead) {
          const uint32_t src = epi_base + ebuf * kEpiStageBytes;
          const int x = x_base + c * EC;
          if (push_all) {
            for (int i = lead_idx; i < W; i += nlead) {  // peers first, starting with the next rank; own copy last
              const int t = (rank + 1 + i) % W;
              if (keeper >= 0 && t != keeper) continue;
              if (p.mode == kEpiReduce) tma_reduce_add_2d(&p.tmC[t], x, y_st, src);
              else if (t == rank && !pulls) tma_store_2d_hint(&p.tmC[t], x, y_st, src, evict_first);
              else tma_store_2d(&p.tmC[t], x, y_st, src);
            }
          } else if (p.mode == kEpiReduce) {
            tma_reduce_add_2d(&p.tmC[rank], x, y_st, src);
          } else if (pulls) {
            tma_store_2d(&p.tmC[rank], x, y_st, src);  // partials are read back soon: keep them in L2
          } else {
            tma_store_2d_hint(&p.tmC[rank], x, y_st, src, evict_first);
          }
          bulk_commit();
          ++groups_this_tile;
        }
        ebuf ^= 1;
      }
      if (++acc == kAccBufs) {
        acc = 0;
        acc_phase ^= 1;
      }
      if (issuer) trace(p, rank, tile * CG + pr, kTrEpiEnd);

      if (pulls) {
        // The partial tile is on its way into this rank's buffer.  Publishing needs its stores to be complete;
        // rather than wait for them now, publish the PREVIOUS tile (its stores are the ones before the up to four
        // groups just committed) and keep this one pending.  The reducer warps do the summing, concurrently.
        if (issuer && !publish_early) {
          if (pending_tile >= 0) {
            // at most the groups just committed may still be pending
            if (groups_this_tile == 4) bulk_wait<4>();
            else if (groups_this_tile == 3) bulk_wait<3>();
            else if (groups_this_tile == 2) bulk_wait<2>();
            else if (groups_this_tile == 1) bulk_wait<1>();
            else bulk_wait<0>();
            publish_tile(pending_tile);
          }
        }
        pending_tile = tile;
      }
    }
    if (pulls && issuer && pending_tile >= 0) {
      bulk_wait<0>();
      publish_tile(pending_tile);
    }
    if (!ok_all && issuer) *abort_flag = 1;

    // Completion: all pushes of this CTA have landed -> bump every rank's arrival counter; then wait until
    // every CTA of every rank has done the same, so that at kernel end all remote tiles are in local memory.
    const bool end_sync = push_all && !pulls;
    if (end_sync) {
      // Every thread that wrote to peers orders its own writes before the arrival the issuer announces below.
      if (direct) {
        fence_sys();
      } else if (lead) {
        bulk_wait<0>();
        fence_proxy_async_all();
        fence_sys();
      }
      named_barrier_sync(1, 128);
      if (issuer) {
        // every writer has fenced at system scope and met this thread at the barrier: one more fence makes that
        // cumulative, and the arrivals themselves can be relaxed (a release per rank would cost a round trip each)
        fence_sys();
        for (int i = 0; i < W; ++i) red_relaxed_sys_add(flag_ptr(p, (rank + 1 + i) % W, 0), 1u);
        if (ok_all) wait_until_ge(flag_ptr(p, rank, 0), callv[2], p.timeout_ns, status, kSiteDone, rank, cta);
      }
    } else if (lead) {
      bulk_wait<0>();
    }
  } else {
    if constexpr (PULL) {
      // ------------------------------------------------------------------------------------------
      // Reducer (128 threads, warps 6-9): sums partial tiles over all ranks while the other warps keep computing.
      // It handles tiles unit, unit + G, ... (two-shot: those this rank owns).  For each, it waits (bounded) for
      // the tile's flag, fetches this CTA's 128 x 256 part as 4 x W units of 128 rows x 64 columns (16 KB) with
      // TMA loads into a ring of pull buffers (a peer's memory included, no multicast), adds in fp32, and writes
      // the bf16 result with TMA stores into the output of this rank (one-shot) or of every rank (two-shot).
      // ------------------------------------------------------------------------------------------
      const int rt = threadIdx.x - 192;
      const bool rissuer = (rt == 0);
      const int row = rt;
      const bool two_shot = p.mode == kEpiTwoShot;
      uint32_t pull_issued = 0, pull_done = 0;  // units issued / consumed so far (ring position)
      bool entered = !(two_shot && W > 1);
      bool ok_all = true;
      float accv[kEpiCols];
      // Sources summed per column chunk: W partial buffers fetched from their owners, or (push_partials) the W x ksplit
      // inbox slots in local memory.  With K-split pieces the unit of reducer work is one column chunk of a tile, so
      // that the summing of a short matrix is spread over as many CTAs as its computation.
      const int ks = p.ksplit > 1 ? p.ksplit : 1;
      const int NS = p.push_partials ? W * ks : W;
      const bool by_chunk = p.ksplit > 1;
      const int kChunks = bn / kEpiCols;
      const int n_items = by_chunk ? total_tiles * kChunks : total_tiles;
      // reduce-scatter: only the tiles of this rank's row block, which are [rank * rs_tpc, (rank + 1) * rs_tpc)
      const int rs_base = p.rs_rows > 0 ? rank * p.rs_rows : 0;
      const int item0 = p.rs_rows > 0 ? rank * rs_tpc + unit : unit;
      const int item_end = p.rs_rows > 0 ? (rank + 1) * rs_tpc : n_items;
      for (int item = item0; item < item_end && ok_all; item += G) {
        const int t = by_chunk ? item / kChunks : item;
        const int c0 = by_chunk ? item - t * kChunks : 0;
        const int c1 = by_chunk ? c0 + 1 : kChunks;
        if (two_shot && owner_of(t) != rank) continue;
        const TileCoord tc = raster(t, tiles_m, tiles_n, p.group_m);
        const int m0 = tc.m_idx * TM + pr * BM, n0 = tc.n_idx * bn;
        if (by_chunk && (n0 + c0 * kEpiCols >= p.N || m0 >= p.M)) continue;
        if (two_shot && p.mc_base != 0 && p.out_row0 >= 0 && W > 1) {
          // NVLS two-shot: the NVLink switch does the work.  One multimem.ld_reduce per 16 bytes returns the fp32-
          // accumulated sum of all W ranks' partials, one multimem.st delivers the result to all W outputs.  A warp
          // covers 512 contiguous bytes (one row of the part) per instruction, eight rows in flight.
          if (rissuer) {
            const uint32_t* f = flag_ptr(p, rank, p.tile_flag_base + t * CG + pr);
            trace(p, rank, t * CG + pr, kTrWaitBegin);
            bool ok = wait_until_ge(f, callv[1], p.timeout_ns, status, kSiteEpiTileFlag, rank, t) == kOk;
            if (ok && !entered) {
              for (int i = 0; i < W && ok; ++i) {
                const int q = (rank + 1 + i) % W;
                ok = wait_until_ge(flag_ptr(p, rank, 8 + q), callv[0], p.timeout_ns, status, kSiteEpiEntry, rank, q) == kOk;
              }
            }
            trace(p, rank, t * CG + pr, kTrWaitEnd);
            *red_ok = ok ? 1u : 0u;
          }
          entered = true;
          named_barrier_sync(3, 128);
          const bool tile_ok = *red_ok != 0;
          named_barrier_sync(3, 128);  // everybody has read the verdict before the issuer writes the next one
          if (!tile_ok) {
            ok_all = false;
            break;
          }
          const int rw = rt >> 5, rl = rt & 31;
          const int col = n0 + rl * 8;
          if (col < p.N && rl * 8 < bn) {
            const uint64_t mc = p.mc_base + p.partial_off;  // [partials | out] matrix of every rank at once
#pragma unroll 1
            for (int r0 = rw * 32; r0 < rw * 32 + 32; r0 += 8) {
              uint4 v[8];
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const int r = m0 + r0 + u;
                if (r < p.M) {
                  const void* src = reinterpret_cast<const void*>(mc + ((uint64_t)((int)callv[3] + r) * p.N + col) * 2);
                  v[u] = f16 ? nvls::ld_reduce_add_f16x8(src) : nvls::ld_reduce_add_bf16x8(src);
                }
              }
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const int r = m0 + r0 + u;
                if (r < p.M)
                  nvls::st_v4(reinterpret_cast<void*>(mc + ((uint64_t)(p.out_row0 + r) * p.N + col) * 2), v[u]);
              }
            }
          }
          if (rissuer) trace(p, rank, t * CG + pr, kTrPullEnd);
          continue;
        }
        if (p.rs_rows > 0) {
          // Reduce-scatter: the W slots of this part are in LOCAL memory and large; rs_sum_part reads them as whole
          // cache lines, adds in fp32 and stores the bf16 rows straight into the kept block (nothing is staged).
          if (rissuer) {
            const uint32_t* f = flag_ptr(p, rank, p.tile_flag_base + t * CG + pr);
            trace(p, rank, t * CG + pr, kTrWaitBegin);
            const bool ok = wait_until_ge(f, callv[1], p.timeout_ns, status, kSiteEpiTileFlag, rank, t) == kOk;
            trace(p, rank, t * CG + pr, kTrWaitEnd);
            *red_ok = ok ? 1u : 0u;
          }
          named_barrier_sync(3, 128);
          const bool part_ok = *red_ok != 0;
          named_barrier_sync(3, 128);  // everybody has read the verdict before the issuer writes the next one
          if (!part_ok) {
            ok_all = false;
            break;
          }
          rs_sum_part(p, rank, NS, m0 - rs_base, n0, rt, f16, (int)callv[3]);
          if (rissuer) trace(p, rank, t * CG + pr, kTrPullEnd);
          continue;
        }
        if (p.push_partials) {
          // Inbox slots are in LOCAL memory: read them with plain coalesced 16-byte loads, many in flight per thread
          // (no ring, no per-unit barriers), add in fp32, and store the chunk through the staging buffer.
          if (rissuer) {
            const uint32_t* f = flag_ptr(p, rank, p.tile_flag_base + t * CG + pr);
            trace(p, rank, t * CG + pr, kTrWaitBegin);
            const bool ok = wait_until_ge(f, callv[1], p.timeout_ns, status, kSiteEpiTileFlag, rank, t) == kOk;
            trace(p, rank, t * CG + pr, kTrWaitEnd);
            *red_ok = ok ? 1u : 0u;
          }
          named_barrier_sync(3, 128);
          const bool tile_ok = *red_ok != 0;
          named_barrier_sync(3, 128);  // everybody has read the verdict before the issuer writes the next one
          if (!tile_ok) {
            ok_all = false;
            break;
          }
          const bool row_live = m0 + row < p.M;
          for (int c = c0; c < c1; ++c) {
            if (n0 + c * kEpiCols >= p.N) break;
#pragma unroll
            for (int j = 0; j < kEpiCols; ++j) accv[j] = 0.f;
            if (row_live) {
              const uint8_t* src = reinterpret_cast<const uint8_t*>(p.heap_base[rank] + p.partial_off) +
                                   ((uint64_t)((int)callv[3] + m0 - rs_base + row) * p.N + n0 + c * kEpiCols) * 2;
              const uint64_t slot_bytes = (uint64_t)p.part_slot_rows * p.N * 2;
              int sl = 0;
              for (; sl + 1 < NS; sl += 2) {
                uint4 v[2][8];
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                  for (int j = 0; j < 8; ++j) v[q][j] = ld_v4(reinterpret_cast<const uint4*>(src + (sl + q) * slot_bytes) + j);
#pragma unroll
                for (int q = 0; q < 2; ++q)
#pragma unroll
                  for (int j = 0; j < 8; ++j) acc_x8(accv + 8 * j, v[q][j], f16);
              }
              for (; sl < NS; ++sl) {
                uint4 v[8];
#pragma unroll
                for (int j = 0; j < 8; ++j) v[j] = ld_v4(reinterpret_cast<const uint4*>(src + sl * slot_bytes) + j);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc_x8(accv + 8 * j, v[j], f16);
              }
            }
            if (p.out_row0 >= 0) {
              if (rissuer) bulk_wait_read<0>();  // the staging buffer's previous store has been read out
              named_barrier_sync(3, 128);
              const uint32_t sbase = redout_base + row * 128;
#pragma unroll
              for (int j = 0; j < 8; ++j)
                st_shared_v4(sbase + ((j ^ (row & 7)) << 4), pack2(accv[8 * j + 0], accv[8 * j + 1], f16),
                             pack2(accv[8 * j + 2], accv[8 * j + 3], f16), pack2(accv[8 * j + 4], accv[8 * j + 5], f16),
                             pack2(accv[8 * j + 6], accv[8 * j + 7], f16));
              fence_proxy_async_smem();
              named_barrier_sync(3, 128);
              if (rissuer) {
                tma_store_2d(&p.tmC[rank], n0 + c * kEpiCols, p.out_row0 + m0 - rs_base, redout_base);
                bulk_commit();
              }
            } else if (row_live) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int col = n0 + c * kEpiCols + 8 * j;
                if (col < p.N) {
                  uint4 o;
                  o.x = pack2(accv[8 * j + 0], accv[8 * j + 1], f16);
                  o.y = pack2(accv[8 * j + 2], accv[8 * j + 3], f16);
                  o.z = pack2(accv[8 * j + 4], accv[8 * j + 5], f16);
                  o.w = pack2(accv[8 * j + 6], accv[8 * j + 7], f16);
                  st_v4(reinterpret_cast<uint4*>(p.heap_base[rank] + p.out_off +
                                                 ((uint64_t)(m0 - rs_base + row) * p.ldo + col) * 2), o);
                }
              }
            }
          }
          if (rissuer) trace(p, rank, t * CG + pr, kTrPullEnd);
          continue;
        }
        const int units = (c1 - c0) * NS;
        auto issue = [&](int u) {  // reducer's issuer only
          const int c = c0 + u / NS, sft = u % NS;
          const uint32_t b = pull_issued % C::kPullBufs;
          mbar_expect_tx(pull_full_bar(b), p.c_box_bytes);
          if (p.push_partials)
            tma_load_2d(pull_base + b * kEpiStageBytes, &p.tmC[rank], n0 + c * kEpiCols,
                        (int)callv[3] + sft * p.part_slot_rows + m0, pull_full_bar(b));
          else
            tma_load_2d(pull_base + b * kEpiStageBytes, &p.tmC[(rank + sft) % W], n0 + c * kEpiCols, (int)callv[3] + m0,
                        pull_full_bar(b));
          ++pull_issued;
        };
        if (rissuer) {
          const uint32_t* f = flag_ptr(p, rank, p.tile_flag_base + t * CG + pr);
          trace(p, rank, t * CG + pr, kTrWaitBegin);
          bool ok = wait_until_ge(f, callv[1], p.timeout_ns, status, kSiteEpiTileFlag, rank, t) == kOk;
          if (ok && !entered) {
            // before the first push of this call: every peer must have entered the call
            for (int i = 0; i < W && ok; ++i) {
              const int q = (rank + 1 + i) % W;
              ok = wait_until_ge(flag_ptr(p, rank, 8 + q), callv[0], p.timeout_ns, status, kSiteEpiEntry, rank, q) == kOk;
            }
          }
          trace(p, rank, t * CG + pr, kTrWaitEnd);
          if (ok) {
            fence_proxy_async_all();  // the flag was acquired with ordinary loads; the data is read by TMA
            for (int u = 0; u < units && u < C::kPullBufs; ++u) issue(u);
            ok = mbar_wait(pull_full_bar(pull_done % C::kPullBufs), (pull_done / C::kPullBufs) & 1, p.timeout_ns,
                           abort_flag);
            if (!ok) record_status(status, kTimeout, kSitePullFull, rank, t, 0);
          }
          *red_ok = ok ? 1u : 0u;
        }
        entered = true;
        for (int u = 0; u < units; ++u) {
          named_barrier_sync(3, 128);  // unit u has landed (or the wait failed): the verdict is in red_ok
          if (*red_ok == 0) {
            ok_all = false;
            break;
          }
          const int c = c0 + u / NS, sft = u % NS;
          const uint32_t buf = pull_base + (pull_done % C::kPullBufs) * kEpiStageBytes + row * 128;
          if (sft == 0) {
#pragma unroll
            for (int j = 0; j < kEpiCols; ++j) accv[j] = 0.f;
          }
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 v;
            asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];"
                         : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(buf + ((j ^ (row & 7)) << 4)));
            acc_x8(accv + 8 * j, v, f16);
          }
          ++pull_done;
          if (sft == NS - 1 && p.out_row0 >= 0) {
            // the result staging buffer must have been read by the previous chunk's stores
            if (rissuer) bulk_wait_read<0>();
          }
          named_barrier_sync(3, 128);  // every thread has read the pull buffer: it can be refilled
          if (rissuer) {
            if (u + C::kPullBufs < units) issue(u + C::kPullBufs);
            if (u + 1 < units) {
              const bool ok = mbar_wait(pull_full_bar(pull_done % C::kPullBufs), (pull_done / C::kPullBufs) & 1,
                                        p.timeout_ns, abort_flag);
              if (!ok) record_status(status, kTimeout, kSitePullFull, rank, t, u + 1);
              *red_ok = ok ? 1u : 0u;
            }
          }
          if (sft != NS - 1) continue;
          if (p.out_row0 >= 0) {
            // Result sub-tile -> swizzled staging buffer -> TMA store: full 128-byte rows on the wire.
            const uint32_t sbase = redout_base + row * 128;
#pragma unroll
            for (int j = 0; j < 8; ++j)
              st_shared_v4(sbase + ((j ^ (row & 7)) << 4), pack2(accv[8 * j + 0], accv[8 * j + 1], f16),
                           pack2(accv[8 * j + 2], accv[8 * j + 3], f16), pack2(accv[8 * j + 4], accv[8 * j + 5], f16),
                           pack2(accv[8 * j + 6], accv[8 * j + 7], f16));
            fence_proxy_async_smem();
            named_barrier_sync(3, 128);
            if (rissuer) {
              const int x = n0 + c * kEpiCols, yy = p.out_row0 + m0;
              if (!two_shot) {
                tma_store_2d(&p.tmC[rank], x, yy, redout_base);
              } else {
                for (int q = 0; q < W; ++q) tma_store_2d(&p.tmC[(rank + 1 + q) % W], x, yy, redout_base);
              }
              bulk_commit();
            }
          } else {
            // the output is a separate buffer of the caller: ordinary 16-byte stores
            const int r = m0 + row;
            if (r < p.M) {
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                const int col = n0 + c * kEpiCols + 8 * j;
                if (col < p.N) {
                  uint4 o;
                  o.x = pack2(accv[8 * j + 0], accv[8 * j + 1], f16);
                  o.y = pack2(accv[8 * j + 2], accv[8 * j + 3], f16);
                  o.z = pack2(accv[8 * j + 4], accv[8 * j + 5], f16);
                  o.w = pack2(accv[8 * j + 6], accv[8 * j + 7], f16);
                  const uint64_t ooff = p.out_off + ((uint64_t)r * p.ldo + col) * 2;
                  if (!two_shot) {
                    st_v4(reinterpret_cast<uint4*>(p.heap_base[rank] + ooff), o);
                  } else {
                    for (int q = 0; q < W; ++q) st_v4(reinterpret_cast<uint4*>(p.heap_base[(rank + 1 + q) % W] + ooff), o);
                  }
                }
              }
            }
          }
        }
        if (rissuer && ok_all) trace(p, rank, t * CG + pr, kTrPullEnd);
      }
      if (!ok_all && rissuer) {
        *abort_flag = 1;
        // fetches already issued still write into the pull buffers: wait, bounded, for each of them
        for (uint32_t i = pull_done; i < pull_issued; ++i)
          mbar_wait(pull_full_bar(i % C::kPullBufs), (i / C::kPullBufs) & 1, 200000, never);
      }
      // Two-shot: when this CTA's pushes have landed, bump every rank's arrival counter and wait (bounded) until
      // every CTA of every rank has done so: at kernel end all result tiles are in local memory.
      if ((two_shot || p.rs_bcast) && W > 1) {
        fence_sys();
        named_barrier_sync(3, 128);
        if (rissuer) {
          bulk_wait<0>();
          fence_proxy_async_all();
          fence_sys();
          for (int i = 0; i < W; ++i) red_relaxed_sys_add(flag_ptr(p, (rank + 1 + i) % W, 0), 1u);
          if (ok_all) wait_until_ge(flag_ptr(p, rank, 0), callv[2], p.timeout_ns, status, kSiteDone, rank, cta);
        }
      } else if (rissuer) {
        bulk_wait<0>();
      }
    } else {
    // ------------------------------------------------------------------------------------------
    // All-gather push (64 threads): this rank's rows of A -> the same rows of every peer's gathered A.
    // ------------------------------------------------------------------------------------------
    if (p.ag && W > 1) {
      const int ct = threadIdx.x - 192;
      const int Ms = p.M / W;
      const int S = p.ag_slices;
      const int slice_elems = p.K / S;             // a multiple of 16 bytes (checked on the host)
      const int vec_per_row = slice_elems * ES / 16;  // 16-byte vectors per row of a slice
      const int items = (W - 1) * chunks_per_shard * S;
      // Nothing is written into a peer's gathered A before that peer has entered this call, i.e. finished the
      // previous one: its producer may otherwise still be loading the rows of the previous call from that buffer.
      if (cta < items) {
        if (ct == 0) {
          bool ok = true;
          for (int i = 0; i + 1 < W && ok; ++i) {
            const int q = (rank + 1 + i) % W;
            ok = wait_until_ge(flag_ptr(p, rank, 8 + q), callv[0], p.timeout_ns, status, kSiteAgEntry, rank, q) == kOk;
          }
          if (!ok) {
            *ag_ok = 0;
            *abort_flag = 1;
          }
        }
        named_barrier_sync(2, 64);
      }
      for (int item = cta; item < items && *ag_ok; item += p.ctas_per_rank) {
        const int pi = item / (chunks_per_shard * S);          // peer-major: finish one peer's copy first
        const int rem = item - pi * (chunks_per_shard * S);
        const int chunk = rem / S;
        const int slice = rem - chunk * S;
        const int peer = (rank - 1 - pi + 2 * W) % W;           // the peer that needs these rows earliest
        const int r0 = rank * Ms + chunk * BM;
        const uint64_t base_off = p.agsrc_off + ((uint64_t)r0 * p.lda_full + (uint64_t)slice * slice_elems) * ES;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(p.heap_base[rank] + base_off);
        uint8_t* dst = reinterpret_cast<uint8_t*>(p.heap_base[peer] + base_off);
        const int nvec = BM * vec_per_row;
        constexpr int kInFlight = 16;  // 16-byte vectors in flight per thread: 16 KB per CTA, enough for link latency
        for (int i0 = ct; i0 < nvec; i0 += 64 * kInFlight) {
          uint4 v[kInFlight];
#pragma unroll
          for (int u = 0; u < kInFlight; ++u) {
            const int i = i0 + u * 64;
            if (i < nvec) {
              const int r = i / vec_per_row, cv = i - r * vec_per_row;
              v[u] = ld_v4(reinterpret_cast<const uint4*>(src + ((uint64_t)r * p.lda_full) * ES + cv * 16));
            }
          }
#pragma unroll
          for (int u = 0; u < kInFlight; ++u) {
            const int i = i0 + u * 64;
            if (i < nvec) {
              const int r = i / vec_per_row, cv = i - r * vec_per_row;
              st_v4(reinterpret_cast<uint4*>(dst + ((uint64_t)r * p.lda_full) * ES + cv * 16), v[u]);
            }
          }
        }
        fence_sys();
        named_barrier_sync(2, 64);
        if (ct == 0) red_release_sys_add(flag_ptr(p, peer, p.ag_flag_base + rank * chunks_per_shard + chunk), 1u);
      }
    }
    }
  }

  // ---- teardown --------------------------------------------------------------------------------
  // Every role that issued bulk copies has waited for them by now: stores with cp.async.bulk.wait_group 0, loads (on
  // the error path) with a bounded wait for the barrier they complete on.
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (p.trace_off && threadIdx.x == 0 && unit < total_tiles) trace(p, rank, tile_of(unit) * CG + pr, kTrCtaEnd);
  if (threadIdx.x == 0) {
    // Call counter: every CTA read it at the start and counts itself here; the last CTA of this rank to arrive makes
    // the call number the new count.  The next launch of this op follows in stream order.
    const uint32_t call = callv[0];
    if (atomicAdd(flag_ptr(p, rank, 3), 1u) + 1u == call * (uint32_t)p.ctas_per_rank)
      *reinterpret_cast<volatile uint32_t*>(flag_ptr(p, rank, 2)) = call;
  }
  if (CG == 2) cluster_sync_all();  // neither CTA of a pair leaves while the other may still touch its memory
  if (warp == 1) {
    __syncwarp();
    if (CG == 1) tmem_dealloc(tmem_base, 512);
    else tmem_dealloc_pair(tmem_base, 512);
  }
}

// ================================================================================================
// Host side
// ================================================================================================
namespace {

thread_local char g_err[512] = "";

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
std::once_flag g_encode_once;

EncodeTiledFn encode_fn() {
  std::call_once(g_encode_once, []() {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      g_encode = reinterpret_cast<EncodeTiledFn>(fn);
    else
      (void)cudaGetLastError();
  });
  return g_encode;
}

// Matrix [rows, cols] of element type `et` (an ElemType) with `ld` elements between rows; box = box_cols x box_rows;
// 128-byte swizzle.
int encode_2d(CUtensorMap* out, uint64_t ptr, uint64_t rows, uint64_t cols, uint64_t ld, uint32_t box_cols,
              uint32_t box_rows, const char* what, int et = kBf16) {
  const uint64_t es = (uint64_t)elem_size(et);
  const CUtensorMapDataType dt = et == kFp16   ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                 : et == kTf32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32
                                 : et == kInt8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                               : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  EncodeTiledFn fn = encode_fn();
  if (!fn) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled is not available");
    return -1;
  }
  if (ptr % 16 != 0 || (ld * es) % 16 != 0) {
    snprintf(g_err, sizeof(g_err), "%s: base address and row pitch must be multiples of 16 bytes", what);
    return -2;
  }
  cuuint64_t dims[2] = {cols, rows};
  cuuint64_t strides[1] = {ld * es};
  cuuint32_t box[2] = {box_cols, box_rows};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(out, dt, 2, reinterpret_cast<void*>(ptr), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_err, sizeof(g_err), "cuTensorMapEncodeTiled(%s) failed with %d", what, (int)r);
    return -3;
  }
  return 0;
}

}  // namespace
}  // namespace gemm
}  // namespace iris

using namespace iris::gemm;

namespace {
using KernelFn = void (*)(const FusedGemmParams);
// The summing (pull) kernels exist for the 16-bit types only; plan creation rejects the other combinations.
KernelFn kernel_for(int cta_group, bool pull, int et) {
  if (et == kTf32) return cta_group == 2 ? fused_gemm_kernel<2, false, kTf32> : fused_gemm_kernel<1, false, kTf32>;
  if (et == kInt8) return cta_group == 2 ? fused_gemm_kernel<2, false, kInt8> : fused_gemm_kernel<1, false, kInt8>;
  if (et == kFp16) {
    if (cta_group == 2) return pull ? fused_gemm_kernel<2, true, kFp16> : fused_gemm_kernel<2, false, kFp16>;
    return pull ? fused_gemm_kernel<1, true, kFp16> : fused_gemm_kernel<1, false, kFp16>;
  }
  if (cta_group == 2) return pull ? fused_gemm_kernel<2, true, kBf16> : fused_gemm_kernel<2, false, kBf16>;
  return pull ? fused_gemm_kernel<1, true, kBf16> : fused_gemm_kernel<1, false, kBf16>;
}
}  // namespace

extern "C" {

// Plain-C description of one fused GEMM; mirrored field by field in iris_b200/ops/gemm.py.
struct IrisGemmDesc {
  uint64_t a_ptr[kMaxRanks];   // per local rank (with ag = 1: the gathered A buffer)
  uint64_t b_ptr[kMaxRanks];   // per local rank
  uint64_t c_ptr[kMaxRanks];   // per target rank: output (store/reduce) or partial buffer parity 0 (one-/two-shot)
  uint64_t c2_ptr[kMaxRanks];  // unused (must be 0): both partial buffers are row ranges of the matrix at c_ptr
  uint64_t heap_base[kMaxRanks];
  int64_t lda[kMaxRanks];      // elements
  int64_t ldb[kMaxRanks];
  int64_t ldc;                 // row pitch of the C / partial buffers
  int64_t c_cols;              // logical number of columns of the C / partial buffers
  int64_t c_rows;              // rows covered by the C tensor maps (0: M)
  uint64_t flags_off;
  uint64_t partial_off[2];
  uint64_t out_off;
  uint64_t status_off;
  uint64_t agsrc_off;
  uint64_t trace_off;
  uint64_t ws_off;
  uint64_t mc_base;
  uint64_t timeout_ns;
  int M, N, K;
  int ldo;
  int part_row0[2];            // per parity
  int out_row0;
  int col_off_per_rank;
  int world, num_local, rank0, ctas_per_rank;
  int mode, group_m, ag, ag_slices, store_all;
  int tile_flag_base, ag_flag_base;
  int device;
  int cta_group;
  int dp_tiles, sk_units, sk_flag_base;  // stream-K schedule (dp_tiles < 0: every tile whole)
  int push_partials, part_slot_rows, ksplit;
  int rs_rows;                 // reduce-scatter: rows kept per rank (0 = off); see FusedGemmParams::rs_rows
  int rs_bcast;                // with rs_rows: the keeper writes the summed rows to every rank's output (all-reduce)
  int bn;                      // tile width: 64, 128 or 256 (0 = 256)
  int dtype;                   // ElemType: 0 = bf16, 1 = fp16, 2 = fp32 as tf32, 3 = int8
  int push_kind;               // PushKind of the all-scatter epilogue
  int tail_tiles, tail_split;  // column-split tail of the raster (see tail_split_plan); 0 / 1 = off
  int sk_slots;                // stream-K: workspace slots per split tile part (1 .. kSkSlots; 0 = kSkSlots)
  uint64_t c_off;              // symmetric offset of the C buffer (needed by push kinds 2 and 3)
  uint64_t zero_bytes;         // atomic all-reduce: bytes of the output (from c_off) the kernel clears itself; 0 = none
};

struct IrisGemmPlan {
  FusedGemmParams params;      // the same for every call: what changes per call is derived in the kernel
  int grid;
  int cooperative;
  int device;
  int cta_group;
  int ctas_per_rank;
  int pull;
  int et;                      // ElemType of the launch
};

// The schedule arithmetic of the kernel, callable on the host (no device needed): see gemm_schedule.h.
void iris_sched_raster(int tile, int tiles_m, int tiles_n, int group_m, int* m_idx, int* n_idx) {
  const TileCoord c = raster(tile, tiles_m, tiles_n, group_m < 1 ? 1 : group_m);
  *m_idx = c.m_idx;
  *n_idx = c.n_idx;
}
int iris_sched_ag_actual_m(int logical_m, int tiles_per_shard, int rank, int world) {
  return ag_actual_m(logical_m, tiles_per_shard, rank, world);
}
int iris_sched_two_shot_owner(int tile, int units, int world) { return two_shot_owner(tile, units, world); }
int iris_sched_sk_unit_of(long long x, long long S, int U) { return sk_unit_of(x, S, U); }
int iris_sched_sk_slots() { return kSkSlots; }
int iris_sched_rs_tile_of(int step, int rank, int world, int tiles_per_block) {
  return rs_tile_of(step, rank, world, tiles_per_block);
}
void iris_sched_tail_split(int total_tiles, int units, int max_split, int* tail_tiles, int* split) {
  tail_split_plan(total_tiles, units, max_split, tail_tiles, split);
}

int iris_sched_work_list_tail(int unit, int units, int total_tiles, int kblocks, int dp_tiles, int sk_units, int ksplit,
                              int tail_tiles, int tail_split, int* out, int max_items, int stride);

// The pieces of work scheduling unit `unit` of `units` goes through, as (tile, kb0, kb1, piece) quadruples; returns how
// many there are (at most `max_items` are written).
int iris_sched_work_list(int unit, int units, int total_tiles, int kblocks, int dp_tiles, int sk_units, int ksplit,
                         int* out, int max_items) {
  return iris_sched_work_list_tail(unit, units, total_tiles, kblocks, dp_tiles, sk_units, ksplit, 0, 1, out, max_items, 4);
}

// The same with a column-split tail; `stride` ints per item: (tile, kb0, kb1, piece[, sub, nsub]).
int iris_sched_work_list_tail(int unit, int units, int total_tiles, int kblocks, int dp_tiles, int sk_units, int ksplit,
                              int tail_tiles, int tail_split, int* out, int max_items, int stride) {
  WorkIter it(unit, units, total_tiles, kblocks, dp_tiles, sk_units, ksplit, tail_tiles, tail_split);
  Work w;
  int n = 0;
  while (it.next(w)) {
    if (n < max_items) {
      out[stride * n] = w.tile;
      out[stride * n + 1] = w.kb0;
      out[stride * n + 2] = w.kb1;
      out[stride * n + 3] = w.piece;
      if (stride >= 6) {
        out[stride * n + 4] = w.sub;
        out[stride * n + 5] = w.nsub;
      }
    }
    ++n;
  }
  return n;
}

const char* iris_gemm_last_error() { return g_err; }
int iris_gemm_smem_bytes() { return kSmemBytes; }
int iris_gemm_desc_size() { return (int)sizeof(IrisGemmDesc); }

void* iris_gemm_plan_create(const IrisGemmDesc* d) {
  g_err[0] = 0;
  if (d->world < 1 || d->world > kMaxRanks || d->num_local < 1 || d->num_local > kMaxRanks) {
    snprintf(g_err, sizeof(g_err), "world and num_local must be in [1, %d]", kMaxRanks);
    return nullptr;
  }
  if (d->M < 1 || d->N < 1 || d->K < 1) {
    snprintf(g_err, sizeof(g_err), "M, N, K must be positive");
    return nullptr;
  }
  if (d->dtype < kBf16 || d->dtype > kInt8) {
    snprintf(g_err, sizeof(g_err), "element type must be bf16 (0), fp16 (1), fp32 multiplied as tf32 (2) or int8 (3)");
    return nullptr;
  }
  const int et = d->dtype;
  const int es = elem_size(et);
  const int epi_cols = 128 / es;  // columns of an epilogue sub-tile (128-byte rows)
  if ((d->N * es) % 16 != 0 || (d->K * es) % 16 != 0) {
    snprintf(g_err, sizeof(g_err), "rows of N and of K elements must be multiples of 16 bytes");
    return nullptr;
  }
  if (d->world > 1 && d->store_all && d->N % epi_cols != 0) {
    snprintf(g_err, sizeof(g_err), "N per rank must be a multiple of %d when tiles are pushed to peers", epi_cols);
    return nullptr;
  }
  if (es != 2 && (d->mode != kEpiStore || d->sk_units > 0 || d->ksplit > 1)) {
    snprintf(g_err, sizeof(g_err), "fp32 and int8 matrices: store mode with whole tiles only (plain GEMM, all-scatter, "
                                   "all-gather prologue)");
    return nullptr;
  }
  const int cg = d->cta_group == 2 ? 2 : 1;
  const int bn = d->bn > 0 ? d->bn : BN;
  if (bn != 64 && bn != 128 && bn != 256) {
    snprintf(g_err, sizeof(g_err), "tile width must be 64, 128 or 256 columns");
    return nullptr;
  }
  if (bn % epi_cols != 0) {
    snprintf(g_err, sizeof(g_err), "tile width must be a multiple of %d columns for this element type", epi_cols);
    return nullptr;
  }
  const int tail_split = d->tail_tiles > 0 && d->tail_split > 1 ? d->tail_split : 1;
  const int tail_tiles = tail_split > 1 ? d->tail_tiles : 0;
  if (tail_split > 1) {
    const bool plain = (d->mode == kEpiStore || d->mode == kEpiReduce) && d->sk_units <= 0 && d->ksplit <= 1;
    if (!plain || bn % tail_split != 0 || (bn / tail_split) % epi_cols != 0 || ((bn / tail_split) / cg) % 8 != 0) {
      snprintf(g_err, sizeof(g_err), "a column-split tail needs store / reduce mode, whole tiles and pieces of whole "
                                     "%d-column sub-tiles", epi_cols);
      return nullptr;
    }
  }
  if (d->push_kind < kPushTma || d->push_kind > kPushMultimem) {
    snprintf(g_err, sizeof(g_err), "push_kind must be 0..3");
    return nullptr;
  }
  if (d->push_kind == kPushStores && d->mode == kEpiReduce) {
    snprintf(g_err, sizeof(g_err), "push_kind 2 (plain stores) cannot add: use 0, 1 or 3 with mode reduce");
    return nullptr;
  }
  if (d->push_kind == kPushMultimem && d->world > 1 && d->store_all &&
      (d->mode == kEpiStore || d->mode == kEpiReduce) && d->mc_base == 0) {
    snprintf(g_err, sizeof(g_err), "push_kind 3 (multimem) needs a heap bound to an NVLS multicast object");
    return nullptr;
  }
  if (d->rs_rows > 0) {
    const int gm = d->group_m < 1 ? 1 : d->group_m;
    if (d->mode != kEpiOneShot || !d->push_partials || d->ksplit > 1 || d->sk_units > 0) {
      snprintf(g_err, sizeof(g_err), "reduce-scatter runs as one-shot with pushed partials, whole tiles, no K split");
      return nullptr;
    }
    if ((long long)d->rs_rows * d->world != d->M || d->rs_rows % (BM * cg) != 0 || (d->rs_rows / (BM * cg)) % gm != 0) {
      snprintf(g_err, sizeof(g_err), "reduce-scatter needs M = world * rs_rows, rs_rows a multiple of %d x group_m",
               BM * cg);
      return nullptr;
    }
    if (d->part_slot_rows < d->rs_rows) {
      snprintf(g_err, sizeof(g_err), "reduce-scatter: inbox slots must hold rs_rows rows");
      return nullptr;
    }
    if (d->rs_bcast && d->out_row0 < 0) {
      snprintf(g_err, sizeof(g_err), "push two-shot: the output must be the symmetric one inside the partial matrix");
      return nullptr;
    }
  }
  if (d->ag) {
    if (d->M % d->world != 0 || (d->M / d->world) % (BM * cg) != 0) {
      snprintf(g_err, sizeof(g_err), "all-gather prologue needs M / world to be a multiple of %d", BM * cg);
      return nullptr;
    }
    if (d->ag_slices < 1 || d->K % d->ag_slices != 0 || (d->K / d->ag_slices * es) % 16 != 0) {
      snprintf(g_err, sizeof(g_err), "ag_slices must divide the rows of K elements into multiples of 16 bytes");
      return nullptr;
    }
  }
  cudaSetDevice(d->device);
  int sms = 0;
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, d->device);
  const bool pull = d->mode == kEpiOneShot || d->mode == kEpiTwoShot;
  for (int t = 0; t < kMaxRanks; ++t) {
    if (d->c2_ptr[t] != 0 || d->partial_off[0] != d->partial_off[1]) {
      snprintf(g_err, sizeof(g_err), "the two partial buffers are row ranges (part_row0) of one matrix per rank");
      return nullptr;
    }
  }
  // Short matrices move short sub-tiles: the C / partial box has only as many rows as M needs (multiple of 8).
  const uint32_t c_box_rows = d->M >= BM ? BM : (uint32_t)((d->M + 7) / 8 * 8);
  int ctas_per_rank = d->ctas_per_rank - d->ctas_per_rank % cg;
  {
    cudaError_t e = cudaFuncSetAttribute(kernel_for(cg, pull, et),
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
    if (e != cudaSuccess) {
      snprintf(g_err, sizeof(g_err), "cudaFuncSetAttribute: %s", cudaGetErrorString(e));
      return nullptr;
    }
  }
  if (cg == 2) {
    // All CTA pairs must be resident at once: ask how many clusters of 2 the device can hold.
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(ctas_per_rank * d->num_local);
    cfg.blockDim = dim3(pull ? kThreadsPull : kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    int max_clusters = 0;
    cudaError_t e = cudaOccupancyMaxActiveClusters(&max_clusters, kernel_for(2, pull, et), &cfg);
    if (e != cudaSuccess || max_clusters < d->num_local) {
      snprintf(g_err, sizeof(g_err), "CTA pairs cannot be scheduled (%s, %d clusters)", cudaGetErrorString(e),
               max_clusters);
      (void)cudaGetLastError();
      return nullptr;
    }
    const int per_rank = 2 * (max_clusters / d->num_local);
    if (ctas_per_rank > per_rank) ctas_per_rank = per_rank;
  }
  const int grid = ctas_per_rank * d->num_local;
  if (ctas_per_rank < 1 || (sms > 0 && grid > sms)) {
    snprintf(g_err, sizeof(g_err), "grid of %d CTAs does not fit %d SMs (all CTAs must be resident)", grid, sms);
    return nullptr;
  }
  IrisGemmPlan* plan = new (std::nothrow) IrisGemmPlan();
  if (!plan) return nullptr;
  memset(plan, 0, sizeof(*plan));
  plan->grid = grid;
  plan->cooperative = d->num_local > 1;
  plan->device = d->device;
  plan->cta_group = cg;
  plan->pull = pull ? 1 : 0;
  plan->et = et;
  plan->ctas_per_rank = ctas_per_rank;
  {
    FusedGemmParams& p = plan->params;
    for (int l = 0; l < d->num_local; ++l) {
      const uint32_t bk = 128 / es;  // K elements of one ring stage: 128 bytes
      if (encode_2d(&p.tmA[l], d->a_ptr[l], d->M, d->K, d->lda[l], bk, BM, "A", et) ||
          encode_2d(&p.tmB[l], d->b_ptr[l], d->N, d->K, d->ldb[l], bk, bn / cg, "B", et) ||
          (tail_split > 1 &&
           encode_2d(&p.tmBt[l], d->b_ptr[l], d->N, d->K, d->ldb[l], bk, (bn / tail_split) / cg, "B (tail)", et))) {
        delete plan;
        return nullptr;
      }
    }
    for (int t = 0; t < d->world; ++t) {
      const uint64_t cp = d->c_ptr[t];
      if (!cp) continue;
      if (encode_2d(&p.tmC[t], cp, d->c_rows > 0 ? d->c_rows : d->M, d->c_cols, d->ldc, epi_cols, c_box_rows, "C",
                    et)) {
        delete plan;
        return nullptr;
      }
    }
    for (int t = 0; t < kMaxRanks; ++t) p.heap_base[t] = d->heap_base[t];
    p.flags_off = d->flags_off;
    p.partial_off = d->partial_off[0];
    p.out_off = d->out_off;
    p.status_off = d->status_off;
    p.agsrc_off = d->agsrc_off;
    p.trace_off = d->trace_off;
    p.c_box_bytes = c_box_rows * 128u;
    p.ws_off = d->ws_off;
    p.mc_base = d->mc_base;
    {
      const int tiles = ((d->M + BM * cg - 1) / (BM * cg)) * ((d->N + bn - 1) / bn);
      p.dp_tiles = (d->dp_tiles < 0 || d->dp_tiles > tiles || d->sk_units <= 0) ? tiles : d->dp_tiles;
      p.sk_units = p.dp_tiles == tiles ? 0 : d->sk_units;
      if (p.sk_units > ctas_per_rank / cg) p.sk_units = ctas_per_rank / cg;  // only units that exist take a range
      if (p.sk_units > 2 * (tiles - p.dp_tiles)) p.sk_units = 2 * (tiles - p.dp_tiles);  // ranges of half a tile or more
      // Slots a split tile needs: the units its k-blocks meet, less the finisher.  The caller sized the workspace for
      // d->sk_slots of them (0: the maximum).
      p.sk_slots = d->sk_slots > 0 ? d->sk_slots : kSkSlots;
      if (p.sk_units > 0) {
        const int kb = (d->K + 128 / es - 1) / (128 / es);
        const long long S = (long long)(tiles - p.dp_tiles) * kb;
        int need = 0;
        for (int t = 0; t < tiles - p.dp_tiles; ++t) {
          const int span =
              sk_unit_of((long long)(t + 1) * kb - 1, S, p.sk_units) - sk_unit_of((long long)t * kb, S, p.sk_units);
          if (span > need) need = span;
        }
        if (need > p.sk_slots || p.sk_slots > kSkSlots) {
          snprintf(g_err, sizeof(g_err), "stream-K: split tiles need %d workspace slots, %d given (at most %d)", need,
                   p.sk_slots, kSkSlots);
          delete plan;
          return nullptr;
        }
      }
      p.sk_flag_base = d->sk_flag_base;
    }
    p.timeout_ns = d->timeout_ns;
    p.M = d->M;
    p.N = d->N;
    p.K = d->K;
    p.ldo = d->ldo;
    p.part_row0 = d->part_row0[0];
    p.part_row0_odd = d->part_row0[1];
    p.per_flag = (uint32_t)(pull ? d->world * (d->ksplit > 1 ? d->ksplit : 1) : d->ag_slices);
    p.out_row0 = d->out_row0;
    p.lda_full = (int)d->lda[0];
    p.col_off_per_rank = d->col_off_per_rank;
    p.world = d->world;
    p.num_local = d->num_local;
    p.rank0 = d->rank0;
    p.ctas_per_rank = ctas_per_rank;
    p.mode = d->mode;
    p.group_m = d->group_m < 1 ? 1 : d->group_m;
    p.ag = d->ag;
    p.ag_slices = d->ag_slices;
    p.store_all = d->store_all;
    p.push_partials = d->push_partials;
    p.part_slot_rows = d->part_slot_rows;
    p.ksplit = d->ksplit > 1 ? d->ksplit : 1;
    p.rs_rows = d->rs_rows > 0 ? d->rs_rows : 0;
    p.rs_bcast = (p.rs_rows > 0 && d->rs_bcast) ? 1 : 0;
    p.tile_flag_base = d->tile_flag_base;
    p.ag_flag_base = d->ag_flag_base;
    p.bn = bn;
    p.dtype = d->dtype;
    p.push_kind = d->push_kind;
    p.tail_tiles = tail_tiles;
    p.tail_split = tail_split;
    p.ldc = (int)d->ldc;
    p.c_off = d->c_off;
    p.zero_bytes = (d->mode == kEpiReduce && d->store_all && d->c_off) ? (d->zero_bytes / 16) * 16 : 0;
  }
  return plan;
}

void iris_gemm_plan_destroy(void* h) { delete static_cast<IrisGemmPlan*>(h); }

// What the plan settled on: CTAs per rank (the done counter advances by world * this per call) and CTA group.
int iris_gemm_plan_ctas_per_rank(void* h) { return static_cast<IrisGemmPlan*>(h)->ctas_per_rank; }
int iris_gemm_plan_cta_group(void* h) { return static_cast<IrisGemmPlan*>(h)->cta_group; }

// Launch one call.  `parity` selects the partial-buffer set; epoch / flag_target / done_target are the
// cumulative values this call drives the flags to (kept by the caller).
// The launch carries no per-call argument (the kernel keeps the call number in device memory), so it may be recorded
// by a stream capture and replayed as part of a CUDA graph.
int iris_gemm_plan_launch(void* h, void* stream) {
  IrisGemmPlan* plan = static_cast<IrisGemmPlan*>(h);
  FusedGemmParams& p = plan->params;
  cudaError_t e;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (plan->cta_group == 2) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan->grid);
    cfg.blockDim = dim3(plan->pull ? kThreadsPull : kThreads);
    cfg.dynamicSmemBytes = kSmemBytes;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeCooperative;
    attr[1].val.cooperative = 1;
    cfg.attrs = attr;
    // Ranks simulated on one GPU wait on one another: ask for a cooperative launch on top of the clusters.
    cfg.numAttrs = plan->cooperative ? 2 : 1;
    void* kargs[] = {&p};
    e = cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kernel_for(2, plan->pull != 0, plan->et)), kargs);
    if (e != cudaSuccess && plan->cooperative) {
      // Cooperative + cluster launches are not accepted everywhere; the grid was sized by
      // cudaOccupancyMaxActiveClusters, so all pairs are resident on an otherwise idle GPU.
      (void)cudaGetLastError();
      cfg.numAttrs = 1;
      e = cudaLaunchKernelExC(&cfg, reinterpret_cast<const void*>(kernel_for(2, plan->pull != 0, plan->et)), kargs);
    }
  } else if (plan->cooperative) {
    void* args[] = {&p};
    e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel_for(1, plan->pull != 0, plan->et)), dim3(plan->grid),
                                    dim3(plan->pull ? kThreadsPull : kThreads), args, kSmemBytes, st);
  } else {
    void* args[] = {&p};
    e = cudaLaunchKernel(reinterpret_cast<void*>(kernel_for(1, plan->pull != 0, plan->et)), dim3(plan->grid),
                         dim3(plan->pull ? kThreadsPull : kThreads), args, kSmemBytes, st);
  }
  if (e != cudaSuccess) {
    snprintf(g_err, sizeof(g_err), "launch failed: %s", cudaGetErrorString(e));
    return -1;
  }
  return 0;
}

}  // extern "C"

// ================================================================================================
// Entry point that allocates nothing (declared and documented in gemm_noalloc.h; no counterpart in the
// reference).  The kernel's scratch is this file-scope device array.  In host code the name `g_noalloc_scratch`
// is only a handle for the runtime's symbol table, NOT a device address: the address the kernel needs is
// obtained once per device with cudaGetSymbolAddress below.
// ================================================================================================
#include "gemm_noalloc.h"

static __device__ __align__(256) unsigned char g_noalloc_scratch[IRIS_GEMM_NOALLOC_SCRATCH_BYTES];

namespace {
constexpr int kNoAllocMaxDevices = 64;
constexpr uint64_t kNoAllocStatusOff = 0;      // iris::StatusBlock (256 bytes reserved)
constexpr uint64_t kNoAllocFlagsOff = 256;     // uint32[16 + max tiles]
constexpr uint64_t kNoAllocPartialOff = IRIS_GEMM_NOALLOC_HEADER_BYTES;  // bf16 [M, N], 256-byte aligned
static_assert(IRIS_GEMM_NOALLOC_HEADER_BYTES % 256 == 0, "partial matrix must stay 256-byte aligned");

struct NoAllocDevice {
  std::atomic<bool> ready{false};    // set (release) after `scratch` and `sms`; read (acquire) without the mutex
  unsigned char* scratch = nullptr;  // device address of g_noalloc_scratch on this device
  int sms = 0;
};
NoAllocDevice g_noalloc_dev[kNoAllocMaxDevices];
std::mutex g_noalloc_mutex;

// Once per device, with that device current.
int noalloc_setup(int dev) {
  std::lock_guard<std::mutex> lock(g_noalloc_mutex);
  NoAllocDevice& d = g_noalloc_dev[dev];
  if (d.ready.load(std::memory_order_acquire)) return 0;
  void* ptr = nullptr;
  cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
  if (e != cudaSuccess || ptr == nullptr) {
    snprintf(iris::gemm::g_err, sizeof(iris::gemm::g_err), "cudaGetSymbolAddress(scratch): %s", cudaGetErrorString(e));
    return -3;
  }
  e = cudaDeviceGetAttribute(&d.sms, cudaDevAttrMultiProcessorCount, dev);
  if (e == cudaSuccess)
    e = cudaFuncSetAttribute(fused_gemm_kernel<1, true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  if (e != cudaSuccess) {
    snprintf(iris::gemm::g_err, sizeof(iris::gemm::g_err), "no-alloc set-up: %s", cudaGetErrorString(e));
    return -3;
  }
  d.scratch = static_cast<unsigned char*>(ptr);
  d.ready.store(true, std::memory_order_release);
  return 0;
}
}  // namespace

extern "C" {

int iris_gemm_noalloc(const void* a, int64_t lda, const void* bt, int64_t ldb, void* out, int64_t ldo, int M, int N,
                      int K, void* stream) {
  char* err = iris::gemm::g_err;
  const size_t errn = sizeof(iris::gemm::g_err);
  err[0] = 0;
  if (!a || !bt || !out || M < 1 || N < 1 || K < 1 || N % 8 != 0 || K % 8 != 0) {
    snprintf(err, errn, "iris_gemm_noalloc: need non-null buffers, positive sizes, N and K multiples of 8");
    return -1;
  }
  if (reinterpret_cast<uintptr_t>(out) % 16 != 0 || (ldo * 2) % 16 != 0 || ldo < N || ldo > 0x7fffffffLL) {
    snprintf(err, errn, "iris_gemm_noalloc: output must be 16-byte aligned with a pitch of N .. 2^31 - 1 elements");
    return -1;
  }
  if (lda < K || ldb < K) {
    snprintf(err, errn, "iris_gemm_noalloc: the row pitches of a and bt must be at least K elements");
    return -1;
  }
  const long long tiles = (long long)((M + BM - 1) / BM) * ((N + BN - 1) / BN);
  if ((unsigned long long)M * (unsigned long long)N > IRIS_GEMM_NOALLOC_MAX_ELEMS ||
      tiles > IRIS_GEMM_NOALLOC_MAX_TILES) {
    snprintf(err, errn,
             "iris_gemm_noalloc: M*N = %lld (%lld tiles) exceeds the built-in scratch (max %u elements, %d tiles); "
             "use the plan-based entry points for larger problems",
             (long long)M * N, tiles, IRIS_GEMM_NOALLOC_MAX_ELEMS, IRIS_GEMM_NOALLOC_MAX_TILES);
    return -2;
  }
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices) {
    snprintf(err, errn, "iris_gemm_noalloc: no current CUDA device");
    return -3;
  }
  if (!g_noalloc_dev[dev].ready.load(std::memory_order_acquire)) {
    const int rc = noalloc_setup(dev);
    if (rc != 0) return rc;
  }
  const NoAllocDevice& d = g_noalloc_dev[dev];
  const uint64_t base = reinterpret_cast<uint64_t>(d.scratch);

  // Parameters live on the host stack; nothing is allocated.
  FusedGemmParams p;
  memset(&p, 0, sizeof(p));
  // a short matrix moves short sub-tiles: the box of the scratch matrix is no taller than M needs (multiple of 8)
  const uint32_t c_box_rows = M >= BM ? BM : (uint32_t)((M + 7) / 8 * 8);
  if (encode_2d(&p.tmA[0], reinterpret_cast<uint64_t>(a), M, K, lda, BK, BM, "A") ||
      encode_2d(&p.tmB[0], reinterpret_cast<uint64_t>(bt), N, K, ldb, BK, BN, "B") ||
      encode_2d(&p.tmC[0], base + kNoAllocPartialOff, M, N, N, kEpiCols, c_box_rows, "scratch partial"))
    return -1;
  p.heap_base[0] = base;                // "heap" of the single rank = the scratch array
  p.flags_off = kNoAllocFlagsOff;
  p.partial_off = kNoAllocPartialOff;
  p.out_off = reinterpret_cast<uint64_t>(out) - base;  // the output is addressed relative to the same base
  p.status_off = kNoAllocStatusOff;
  p.timeout_ns = 2000000000ull;
  p.M = M;
  p.N = N;
  p.K = K;
  p.ldo = (int)ldo;
  p.c_box_bytes = c_box_rows * 128u;
  p.part_row0 = p.part_row0_odd = 0;
  p.per_flag = 1;  // one rank raises each tile's flag once; the flags (call counter included) are cleared just below
  p.out_row0 = -1;  // the caller's output is a separate buffer: ordinary stores
  p.world = 1;
  p.num_local = 1;
  p.rank0 = 0;
  p.ctas_per_rank = (int)(tiles < d.sms ? tiles : d.sms);
  p.mode = kEpiOneShot;
  p.ksplit = 1;
  p.group_m = 8;
  p.dp_tiles = (int)tiles;  // every tile is computed whole by one CTA
  p.sk_units = 0;
  p.tile_flag_base = 16;
  p.ag_flag_base = 16;
  p.bn = BN;
  p.dtype = kBf16;
  p.tail_split = 1;

  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // The scratch keeps the previous call's contents.  The per-tile flags have to start at zero: clear them in stream
  // order.  The status record is left alone, so that a time-out of an earlier call stays readable until
  // iris_gemm_noalloc_status() has reported it.
  cudaError_t e = cudaMemsetAsync(d.scratch + kNoAllocFlagsOff, 0, (size_t)(16 + tiles) * sizeof(uint32_t), st);
  if (e == cudaSuccess) {
    fused_gemm_kernel<1, true, kBf16><<<p.ctas_per_rank, kThreadsPull, kSmemBytes, st>>>(p);
    e = cudaGetLastError();
  }
  if (e != cudaSuccess) {
    snprintf(err, errn, "iris_gemm_noalloc: %s", cudaGetErrorString(e));
    return -3;
  }
  return 0;
}

int iris_gemm_noalloc_status(void) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kNoAllocMaxDevices ||
      !g_noalloc_dev[dev].ready.load(std::memory_order_acquire))
    return 0;
  if (cudaDeviceSynchronize() != cudaSuccess) return -3;
  unsigned char* st = g_noalloc_dev[dev].scratch + kNoAllocStatusOff;
  uint32_t code = 0;
  if (cudaMemcpy(&code, st, sizeof(code), cudaMemcpyDeviceToHost) != cudaSuccess) return -3;
  // reported once: the record is cleared so that it describes the calls made after this one
  if (code != 0 && cudaMemset(st, 0, sizeof(iris::StatusBlock)) != cudaSuccess) return -3;
  return (int)code;
}

}  // extern "C"
