// gemm_fused.cuh — parameters shared by the host launcher and the device code of the fused
// GEMM + collective kernels (gemm_fused.cu).
//
// One kernel family replaces the reference's three Triton kernels:
//   * examples/07_gemm_all_scatter/gemm_all_scatter.py:97-255        -> kEpiStore   (push tile to every rank)
//   * examples/08_gemm_atomics_all_reduce/gemm_atomics_all_reduce.py:94-252 -> kEpiReduce (add tile into every rank)
//   * examples/09_gemm_one_shot_all_reduce/gemm_one_shot_all_reduce.py:94-275 -> kEpiOneShot / kEpiTwoShot
// plus the all-gather -> GEMM prologue, the push / K-split form of one-shot for short matrices and the NVLS two-shot
// reducer, which the reference does not have.
#pragma once
#include <cuda.h>
#include <stdint.h>

namespace iris {
namespace gemm {

constexpr int kMaxRanks = 8;

// Tile shape of one CTA: 128 rows x up to 256 columns of output, 64-deep K slices (128 bytes of a 16-bit type: one
// swizzle row).  The width actually used is a launch parameter (FusedGemmParams::bn: 64, 128 or 256); BN is the
// widest, for which shared memory and tensor memory are laid out.
constexpr int BM = 128;
constexpr int BN = 256;
constexpr int BK = 64;
constexpr int UMMA_K = 16;
constexpr int kStages = 4;   // shared-memory ring of (A,B) slices for single CTAs (see Cfg in gemm_fused.cu for the others)
constexpr int kAccBufs = 2;  // TMEM accumulators: epilogue of tile i overlaps main loop of tile i+1
constexpr int kEpiCols = 64; // epilogue works on 128 x 64 sub-tiles (128-byte rows of bf16)
constexpr int kEpiBufs = 2;

constexpr int kAStageBytes = BM * BK * 2;
constexpr int kBStageBytes = BN * BK * 2;
constexpr int kStageBytes = kAStageBytes + kBStageBytes;
constexpr int kEpiStageBytes = BM * kEpiCols * 2;
constexpr int kSmemTiles = kStages * kStageBytes + kEpiBufs * kEpiStageBytes;
constexpr int kSmemBarriers = 256;
constexpr int kSmemBytes = kSmemTiles + kSmemBarriers + 1024;  // + slack to align the base to 1024 B

// Slots of one per-tile trace record (nanoseconds of the global timer).
enum TraceSlot : int { kTrMmaBegin = 0, kTrMmaEnd = 1, kTrEpiBegin = 2, kTrEpiEnd = 3, kTrWaitBegin = 4, kTrWaitEnd = 5,
                       kTrPullEnd = 6, kTrCtaBegin = 7, kTrCtaEnd = 8, kTrSlots = 10 };

constexpr int kThreads = 256;      // warp 0: TMA producer, warp 1: MMA issuer, warps 2-5: epilogue, warps 6-7: all-gather push
constexpr int kThreadsPull = 320;  // one-/two-shot kernels: warps 6-9 are the reducer (pull, sum, write) instead

// How a finished tile reaches the other ranks in store mode with store_all (GEMM + all-scatter).
enum PushKind : int {
  kPushTma = 0,       // one thread issues a TMA store per destination rank
  kPushTmaSpread = 1, // the four epilogue warp leaders share the destination ranks
  kPushStores = 2,    // all 128 epilogue threads copy the staged sub-tile with 16-byte stores, a row segment per 8 lanes
  kPushMultimem = 3,  // as kPushStores, but ONE multimem.st per 16 bytes: the NVLink switch delivers it to every rank
};

// Element type of A, B and C.  bf16 / fp16: fp32 accumulation.  kTf32: fp32 matrices, multiplied as tf32 (10-bit
// mantissa) with fp32 accumulation.  kInt8: signed 8-bit matrices, 32-bit integer accumulation, and the low 8 bits
// of the sum as the result (two's-complement wrap, what a cast of the accumulator to int8 gives).  The 32- and 8-bit
// types exist for the store mode only (plain GEMM, GEMM + all-scatter, all-gather + GEMM).
enum ElemType : int { kBf16 = 0, kFp16 = 1, kTf32 = 2, kInt8 = 3 };
__host__ __device__ constexpr int elem_size(int et) { return et == kTf32 ? 4 : et == kInt8 ? 1 : 2; }

enum EpiMode : int {
  kEpiStore = 0,    // C tile -> TMA store into the C buffer of every rank (world 1: plain GEMM)
  kEpiReduce = 1,   // C tile -> TMA reduce-add into the C buffer of every rank (C must start at zero)
  kEpiOneShot = 2,  // partial tile -> own partial buffer; flags; every rank pulls all partials and sums
  kEpiTwoShot = 3,  // as one-shot, but tile t is summed only by rank t % world, which pushes the result
};

struct FusedGemmParams {
  // Tensor maps (host-encoded).  Index = local rank for A and B, target rank for C.
  CUtensorMap tmA[kMaxRanks];  // [rows M, cols K] bf16, K contiguous, box 64 x 128, 128-byte swizzle
  CUtensorMap tmB[kMaxRanks];  // [rows N, cols K] bf16, K contiguous, box 64 x (bn / cta group), 128-byte swizzle
  CUtensorMap tmBt[kMaxRanks]; // the same matrix with the shorter box of a tail tile's column piece
  CUtensorMap tmC[kMaxRanks];  // [rows M, cols ldc] bf16, box 64 x 128, 128-byte swizzle
                               //   store/reduce: the output of rank t; one-/two-shot: the partial buffer of rank t
  uint64_t heap_base[kMaxRanks];  // base address of every rank's heap in this process
  // Symmetric offsets (bytes from the heap base) of the communication state.
  uint64_t flags_off;    // uint32[...]: [0] arrival counter, [8 + r] entry flag of rank r, then per-tile /
                         // per-chunk flags at tile_flag_base / ag_flag_base
  uint64_t partial_off;  // one-/two-shot: bf16 [M, N] partial buffer of the current parity
  uint64_t out_off;      // one-/two-shot: bf16 [M, ldo] final output
  uint64_t status_off;   // iris::StatusBlock
  uint64_t agsrc_off;    // all-gather prologue: gathered A [M, K] (row stride lda_full elements)
  uint64_t mc_base;      // NVLS multicast address of the heap (0: not bound); used by the two-shot reducer
  uint64_t ws_off;       // stream-K: fp32 workspace [split tiles * cta_group][128][256] per rank, zero between calls
  uint64_t trace_off;    // 0, or int64[tiles * cta_group][8] per rank: per-tile device timestamps (ns)
  uint64_t timeout_ns;
  int M, N, K;           // per-rank GEMM problem: C[M, N] = A[M, K] * B[N, K]^T
  int part_row0;         // one-/two-shot: first row, inside the tmC matrices, of this call's partial buffer
  int out_row0;          // one-/two-shot: first row of the final output inside the tmC matrices, or -1 when the
                         // output is a separate buffer written with ordinary stores (out_off, ldo)
  int ldo;               // row stride (elements) of the final output in one-/two-shot mode
  int lda_full;          // row stride (elements) of the gathered A
  int col_off_per_rank;  // store/reduce: rank r writes columns [r * col_off_per_rank, ... + N) of C
  int world;             // ranks taking part in the collective
  int num_local;         // ranks simulated by this launch (1 on real multi-GPU runs)
  int rank0;             // rank of local index 0
  int ctas_per_rank;
  int mode;              // EpiMode
  int group_m;           // raster: m-tiles per group
  int ag;                // 1: A is gathered by the comm warps of this kernel (rows sharded M / world per rank)
  int ag_slices;         // column slices per 128-row chunk in the all-gather push
  int dp_tiles;          // tiles [0, dp_tiles) are computed whole (tile = unit + i * units); the others are split
                         // by k-blocks over `sk_units` scheduling units (stream-K), 0 = no split tiles
  int sk_units;
  int sk_flag_base;      // index of the per-(split tile, CTA of the group) counters of parked pieces
  int sk_slots;          // workspace slots per split tile part (stride of the workspace; at most kSkSlots)
  int push_partials;     // one-shot: 1 = every rank's partial tile is pushed into a slot of every rank's inbox and summed
                         // from local memory; 0 = partials stay home and are fetched by the reducers
  int part_slot_rows;    // rows between consecutive inbox slots inside the tmC matrices
  int ksplit;            // one-shot with push: each tile's K range is cut into `ksplit` pieces computed by different
                         // CTAs, each piece a slot of its own (slot = rank * ksplit + piece); 1 = no split
  int rs_rows;           // one-shot with push, reduce-scatter: > 0 = rank r keeps only rows [r * rs_rows, (r + 1) * rs_rows)
                         // of the sum.  A partial tile goes to the inbox of the rank that keeps its rows only (slot = source
                         // rank, rows relative to the keeper's first row); rank r takes successive tiles from the row blocks
                         // r + 1, r + 2, ..., r in turn, so that at any time every keeper is receiving from one source.  0 = off
  int rs_bcast;          // with rs_rows: the keeper writes every summed row to the output of ALL ranks (the output then has
                         // all M rows): GEMM + all-reduce as reduce-scatter by pushes + broadcast ("push two-shot")
  int store_all;         // store/reduce modes: 1 = push the tile to every rank, 0 = own rank only
  int tile_flag_base;    // index (uint32 units from flags_off) of the per-tile flags
  int ag_flag_base;      // index of the all-gather chunk flags: [src rank][chunk]
  int bn;                // tile width in columns: 64, 128 or 256 (multiple of 64)
  int dtype;             // ElemType of A, B, C
  int push_kind;         // PushKind (store mode with store_all)
  int tail_tiles;        // the last `tail_tiles` tiles of the raster are cut into `tail_split` column pieces each
  int tail_split;        //   (see tail_split_plan in gemm_schedule.h); 0 / 1 = no split
  int ldc;               // row pitch (elements) of the C buffers, for the pushes made with ordinary / multimem stores
  uint64_t c_off;        // symmetric offset of the C buffer (store / reduce with store_all)
  uint64_t zero_bytes;   // reduce mode: bytes of this rank's output, from c_off, that the kernel clears before it
                         // raises its entry flags (multiple of 16; 0 = the caller clears the output)
  uint32_t c_box_bytes;  // bytes of one C / partial sub-tile transfer: rows of the tmC box (128, fewer when M < 128) x 128
  // Nothing in the launch arguments changes from call to call: the call number is kept in device memory (flag
  // word [2]: calls completed, written by the last CTA of a launch to leave, counted on word [3]) and everything
  // that depends on it is derived in the kernel: the value of the entry flags (the call number), what the
  // cumulative per-tile / per-chunk flags reach in this call (per_flag x call), what the arrival counter reaches
  // (call x world x CTAs per rank), and which of the two partial buffers is written (call parity).  A launch can
  // therefore be recorded in a CUDA graph and replayed.
  uint32_t per_flag;     // what one call adds to a per-tile flag (ranks x K pieces) or to a per-chunk flag (slices)
  int part_row0_odd;     // part_row0 of odd-numbered calls (part_row0 above: even-numbered calls)
};

}  // namespace gemm
}  // namespace iris
