// attention.cu — causal (or full) self-attention forward for head dimension 128 on the 5th-generation tensor cores.
//
//   O[b, s, h, :] = softmax(Q[b, s, h, :] . K[b, 0..s, h, :]^T / sqrt(128)) . V[b, 0..s, h, :]
//
// Q, K and V are the three column blocks of ONE matrix qkv[T = B * S, 3 * heads * 128] (the output of the fused
// all-gather -> GEMM of the tensor-parallel decoder block), O is [T, heads * 128]; 16-bit elements (bf16 or fp16),
// fp32 accumulation and softmax.  No counterpart in the reference (it has no model code); it replaces the library
// attention call inside iris_b200/models/tp_block.py.
//
// One CTA per (batch, head, tile of 128 queries); it walks over the key tiles of 128 (causal: up to its own):
//   warp 0      TMA producer: Q once, then K_j / V_j into a two-stage ring (cp.async.bulk.tensor, no multicast)
//   warp 1      one thread issues tcgen05.mma:  S_j = Q K_j^T (128 x 128 x 128, both operands K-major) into one of
//               two S accumulators in tensor memory, and O_j = P_j V_j (P from shared memory, V as an MN-major
//               operand: V[key][d] is read as stored) into one of two O accumulators
//   warps 2-9   softmax, two threads per query row (64 keys / 64 output columns each): tcgen05.ld of S_j, running
//               maximum (over the whole row, read by both), exp2, row sum, P_j as 16-bit values into shared
//               memory in the swizzled layout the MMA expects; then O_{j-1} is read from tensor memory and folded
//               into the fp32 output row kept in registers (rescaled by exp2(m_old - m_new)).
// While the softmax warps work on S_j the tensor cores already compute S_{j+1}.
//
// Every wait is bounded by timeout_ns: on expiry the CTA records a status, every role leaves its loop, tensor memory
// is released and the kernel returns.
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <mutex>

#include "iris/iris.cuh"
#include "iris/ptx_sm100.cuh"

namespace iris {
namespace attn {

using namespace iris::ptx;

constexpr int D = 128;            // head dimension
constexpr int BQ = 128;           // queries per CTA
constexpr int BKV = 128;          // keys per tile
constexpr int kTileBytes = 128 * 128 * 2;   // one 128 x 128 tile of 16-bit elements (two 64-column swizzle blocks)
constexpr int kHalfBytes = kTileBytes / 2;  // one 64-column block: 128 rows x 128 bytes
constexpr int kThreads = 320;          // TMA warp, MMA warp, eight softmax warps
// shared memory: Q | K[2] | V[2] | P, then barriers
constexpr int kSmemTiles = 6 * kTileBytes;
constexpr int kXchgBytes = 256 * 4;         // row sums exchanged between the two halves at the end
constexpr int kSmemBytes = kSmemTiles + 256 + kXchgBytes + 1024;

enum Site : uint32_t { kSiteLoad = 90, kSiteMma = 91, kSiteSoftmax = 92 };

// 2^x on the special-function unit (ex2.approx: 2 ulp, 2^-inf = 0), which is what bounds the softmax warps.
__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct Params {
  CUtensorMap tm;        // qkv [T, 3 * heads * 128], box 64 columns x 128 rows, 128-byte swizzle
  void* out;             // [T, heads * 128]
  int64_t ldo;           // row pitch of out, elements
  StatusBlock* status;
  uint64_t timeout_ns;
  int batch, seq, heads;
  int causal;
  float scale_log2;      // log2(e) / sqrt(128)
};

template <bool F16>
__global__ void __launch_bounds__(kThreads, 1) attention_fwd_kernel(const __grid_constant__ Params p) {
  constexpr int kFirstSoftmaxWarp = 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const uint32_t q_s = smem_u32(smem);
  const uint32_t k_s = q_s + kTileBytes;          // 2 stages
  const uint32_t v_s = k_s + 2 * kTileBytes;      // 2 stages
  const uint32_t p_s = v_s + 2 * kTileBytes;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + kSmemTiles);
  const uint32_t bar0 = smem_u32(bars);
  // 0 q_full | 1,2 k_full | 3,4 v_full | 5,6 kv_empty | 7,8 s_full | 9,10 s_free | 11 p_ready | 12,13 o_full | 14,15 o_free
  auto bar = [&](int i) { return bar0 + 8u * i; };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(bars + 16);
  volatile uint32_t* abort_flag = tmem_slot + 1;
  volatile float* xchg = reinterpret_cast<volatile float*>(smem + kSmemTiles + 256);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = p.seq / BQ;
  const int bh = blockIdx.x % (p.batch * p.heads);
  const int qt = nq - 1 - blockIdx.x / (p.batch * p.heads);   // longest rows of work first
  const int b = bh / p.heads, h = bh - b * p.heads;
  const int nkv = p.causal ? qt + 1 : p.seq / BKV;
  const int row0 = b * p.seq + qt * BQ;           // first query row in the [T, ...] matrices
  const int xq = h * D, xk = (p.heads + h) * D, xv = (2 * p.heads + h) * D;

  if (threadIdx.x == 0) {
    for (int i = 0; i < 16; ++i) {
      const bool by_warps = (i == 9 || i == 10 || i == 11 || i == 14 || i == 15);  // one arrival per softmax warp
      mbar_init(bar(i), by_warps ? 8 : 1);
    }
    *abort_flag = 0;
    mbar_fence_init();
    prefetch_tensormap(&p.tm);
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), 512);   // S[2] and O[2], 128 columns each
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp == 0) {
    if (lane == 0) {
      mbar_expect_tx(bar(0), kTileBytes);
      tma_load_2d(q_s, &p.tm, xq, row0, bar(0));
      tma_load_2d(q_s + kHalfBytes, &p.tm, xq + 64, row0, bar(0));
      for (int j = 0; j < nkv; ++j) {
        const int st = j & 1;
        if (j >= 2 && !mbar_wait(bar(5 + st), ((j >> 1) - 1) & 1, p.timeout_ns, abort_flag)) {
          record_status(p.status, kTimeout, kSiteLoad, blockIdx.x, j, 0);
          *abort_flag = 1;
          break;
        }
        const int krow = b * p.seq + j * BKV;
        mbar_expect_tx(bar(1 + st), kTileBytes);
        tma_load_2d(k_s + st * kTileBytes, &p.tm, xk, krow, bar(1 + st));
        tma_load_2d(k_s + st * kTileBytes + kHalfBytes, &p.tm, xk + 64, krow, bar(1 + st));
        mbar_expect_tx(bar(3 + st), kTileBytes);
        tma_load_2d(v_s + st * kTileBytes, &p.tm, xv, krow, bar(3 + st));
        tma_load_2d(v_s + st * kTileBytes + kHalfBytes, &p.tm, xv + 64, krow, bar(3 + st));
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      constexpr uint32_t idesc_qk = umma_idesc_f16_major(BQ, BKV, !F16, false, false);
      constexpr uint32_t idesc_pv = umma_idesc_f16_major(BQ, D, !F16, false, true);   // V is MN-major
      bool ok = true;
      auto fail = [&](int j, int what) {
        record_status(p.status, kTimeout, kSiteMma, blockIdx.x, j, what);
        *abort_flag = 1;
        ok = false;
      };
      // S_j = Q K_j^T into S accumulator j & 1
      auto issue_qk = [&](int j) {
        const int st = j & 1;
        if (!mbar_wait(bar(1 + st), (j >> 1) & 1, p.timeout_ns, abort_flag)) return fail(j, 1);
        if (j >= 2 && !mbar_wait(bar(9 + st), ((j >> 1) - 1) & 1, p.timeout_ns, abort_flag)) return fail(j, 2);
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * kHalfBytes + (kk & 3) * 32;
          umma_f16_ss(tmem + st * 128, umma_desc_k_sw128(q_s + off), umma_desc_k_sw128(k_s + st * kTileBytes + off),
                      idesc_qk, kk ? 1u : 0u);
        }
        umma_commit(bar(7 + st));
      };
      if (!mbar_wait(bar(0), 0, p.timeout_ns, abort_flag)) fail(0, 0);
      if (ok) issue_qk(0);
      for (int j = 0; j < nkv && ok; ++j) {
        const int st = j & 1;
        if (j + 1 < nkv) issue_qk(j + 1);
        if (!ok) break;
        if (!mbar_wait(bar(11), j & 1, p.timeout_ns, abort_flag)) { fail(j, 3); break; }          // P_j in shared memory
        if (!mbar_wait(bar(3 + st), (j >> 1) & 1, p.timeout_ns, abort_flag)) { fail(j, 4); break; }  // V_j loaded
        if (j >= 2 && !mbar_wait(bar(14 + st), ((j >> 1) - 1) & 1, p.timeout_ns, abort_flag)) { fail(j, 5); break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < BKV / 16; ++kk) {
          const uint64_t a_desc = umma_desc_k_sw128(p_s + (kk >> 2) * kHalfBytes + (kk & 3) * 32);
          // 16 keys = two groups of 8 rows (1024 bytes apart); the second 64 columns of d are one half tile further on
          const uint64_t b_desc = umma_desc_mn_sw128(v_s + st * kTileBytes + kk * 16 * 128, kHalfBytes, 1024);
          umma_f16_ss(tmem + 256 + st * 128, a_desc, b_desc, idesc_pv, kk ? 1u : 0u);
        }
        umma_commit(bar(12 + st));   // O_j complete (and P free again)
        umma_commit(bar(5 + st));    // K_j / V_j stage free
      }
    }
  } else if (warp >= kFirstSoftmaxWarp) {
    // ---- softmax + output: two threads per query row, one for keys / output columns 0..63, one for 64..127 ----
    // (a warp may only read the 32 tensor-memory lanes of its quadrant, warp id % 4; warps 2-5 take the first half of
    // the columns, warps 6-9 the second, so that every scheduler of the SM has two softmax warps to switch between)
    const int quad = warp & 3;
    const int half = (warp - kFirstSoftmaxWarp) >> 2;
    const int row = quad * 32 + lane;
    const uint32_t lane_addr = (uint32_t)(quad * 32) << 16;
    float acc[64];
#pragma unroll
    for (int i = 0; i < 64; ++i) acc[i] = 0.f;
    float m_run = -INFINITY, l_run = 0.f, alpha_prev = 0.f;   // l_run: this half's part of the row sum
    bool ok = true;
    auto fail = [&](int j, int what) {
      if (lane == 0) record_status(p.status, kTimeout, kSiteSoftmax, blockIdx.x, j, what);
      *abort_flag = 1;
      ok = false;
    };
    // fold this thread's 64 columns of O_j (accumulator j & 1) into its output row: acc = acc * alpha + O_j
    auto fold_o = [&](int j, float alpha) {
      const int st = j & 1;
      if (!mbar_wait(bar(12 + st), (j >> 1) & 1, p.timeout_ns, abort_flag)) return fail(j, 2);
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {   // 32 columns at a time: the row of S or O is never whole in registers
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + 256 + st * 128 + half * 64 + c * 32, v);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) acc[c * 32 + i] = acc[c * 32 + i] * alpha + __uint_as_float(v[i]);
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(bar(14 + st));
    };
    for (int j = 0; j < nkv; ++j) {
      const int st = j & 1;
      if (!mbar_wait(bar(7 + st), (j >> 1) & 1, p.timeout_ns, abort_flag)) fail(j, 1);
      const bool diag = p.causal && j == qt;
      if (!ok) break;
      // pass 1: maximum of the WHOLE row of scores (both halves: two more tensor-memory loads are cheaper than an
      // exchange through shared memory and a barrier of all softmax warps in every tile)
      float mx = -INFINITY;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem + lane_addr + st * 128 + c * 32, v);
        tmem_wait_ld();
        if (diag) {   // keys after the query: minus infinity (ignored by the maximum, 0 after the exponential)
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i > row) v[i] = 0xff800000u;
        }
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four chains instead of one long one
#pragma unroll
        for (int i = 0; i < 32; ++i) m4[i & 3] = fmaxf(m4[i & 3], __uint_as_float(v[i]));
        mx = fmaxf(mx, fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));
      }
      const float m_new = fmaxf(m_run, mx * p.scale_log2);
      const float alpha = fast_exp2(m_run - m_new);       // 0 for the first tile (m_run = -inf)
      // P overwrites the buffer the previous P V product reads: that product must have completed
      if (j >= 1 && !mbar_wait(bar(12 + ((j - 1) & 1)), ((j - 1) >> 1) & 1, p.timeout_ns, abort_flag)) fail(j, 3);
      float sum = 0.f;
      float s4[4] = {0.f, 0.f, 0.f, 0.f};
      if (ok) {
        // keys half*64 .. +63 of this row = 64-key block `half`, eight 16-byte pieces, swizzled by the row
        const uint32_t base = p_s + half * kHalfBytes + row * 128;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {   // pass 2, 32 scores at a time
          uint32_t v[32];
          tmem_ld_32x32b_x32(tmem + lane_addr + st * 128 + half * 64 + c2 * 32, v);
          tmem_wait_ld();
          if (diag) {
#pragma unroll
            for (int i = 0; i < 32; ++i)
              if (half * 64 + c2 * 32 + i > row) v[i] = 0xff800000u;
          }
#pragma unroll
          for (int qq = 0; qq < 4; ++qq) {
            const int q = c2 * 4 + qq;       // 16-byte piece (8 keys) of this thread's 64 keys
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const int c = qq * 8 + 2 * i;  // index inside v
              float e0 = fast_exp2(__uint_as_float(v[c]) * p.scale_log2 - m_new);
              float e1 = fast_exp2(__uint_as_float(v[c + 1]) * p.scale_log2 - m_new);
              s4[i] += e0 + e1;
              if (F16) {
                __half2 hh = __floats2half2_rn(e0, e1);
                pk[i] = *reinterpret_cast<uint32_t*>(&hh);
              } else {
                __nv_bfloat162 bb = __floats2bfloat162_rn(e0, e1);
                pk[i] = *reinterpret_cast<uint32_t*>(&bb);
              }
            }
            asm volatile("st.shared.v4.u32 [%0], {%1,%2,%3,%4};" ::"r"(base + ((q ^ (row & 7)) << 4)), "r"(pk[0]),
                         "r"(pk[1]), "r"(pk[2]), "r"(pk[3])
                         : "memory");
          }
        }
        sum = (s4[0] + s4[1]) + (s4[2] + s4[3]);
        l_run = l_run * alpha + sum;
        m_run = m_new;
        fence_proxy_async_smem();   // P is read by the tensor core through the async proxy
        tc_fence_before();
        __syncwarp();
        if (lane == 0) {
          mbar_arrive(bar(11));        // this warp's part of P_j is in shared memory
          mbar_arrive(bar(9 + st));    // and it has finished reading the S accumulator
        }
        if (j >= 1) fold_o(j - 1, alpha_prev);
        alpha_prev = alpha;
      }
    }
    if (ok) fold_o(nkv - 1, alpha_prev);
    // total row sum = the two halves' sums
    xchg[half * 128 + row] = ok ? l_run : NAN;
    named_barrier_sync(1, 256);
    const float l_other = xchg[(half ^ 1) * 128 + row];
    if (ok && l_other == l_other) {
      const float inv = 1.f / (l_run + l_other);
      uint8_t* orow = reinterpret_cast<uint8_t*>(p.out) +
                      ((int64_t)(row0 + row) * p.ldo + (int64_t)h * D + half * 64) * 2;
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4 o;
        uint32_t* w = reinterpret_cast<uint32_t*>(&o);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float a = acc[c * 8 + 2 * i] * inv, bb = acc[c * 8 + 2 * i + 1] * inv;
          if (F16) {
            __half2 hh = __floats2half2_rn(a, bb);
            w[i] = *reinterpret_cast<uint32_t*>(&hh);
          } else {
            __nv_bfloat162 t = __floats2bfloat162_rn(a, bb);
            w[i] = *reinterpret_cast<uint32_t*>(&t);
          }
        }
        *reinterpret_cast<uint4*>(orow + c * 16) = o;
      }
    }
  }

  // ---- teardown: loads still in flight on the error path are given their barrier (bounded) ----
  __syncwarp();
  if (*abort_flag && warp == 0 && lane == 0) {
    volatile uint32_t never = 0;
    for (int i = 0; i < 5; ++i) mbar_wait(bar(i), 0, 50000, &never);
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    __syncwarp();
    tmem_dealloc(tmem, 512);
  }
}

}  // namespace attn
}  // namespace iris

// ================================================================================================
// Host side
// ================================================================================================
namespace {
thread_local char g_attn_err[256] = "";

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn attn_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, []() {
    void* q = nullptr;
    cudaDriverEntryPointQueryResult r;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &q, cudaEnableDefault, &r) == cudaSuccess &&
        r == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(q);
    else
      (void)cudaGetLastError();
  });
  return fn;
}
}  // namespace

extern "C" {

const char* iris_attention_last_error() { return g_attn_err; }

// qkv: [batch * seq, 3 * heads * 128] (row pitch ld_qkv elements): columns [0, heads*128) are Q, the next heads*128 K,
// the last heads*128 V, head h in columns h*128 .. of each block.  out: [batch * seq, heads * 128] (row pitch ldo).
// dtype: 0 = bf16, 1 = fp16.  seq must be a multiple of 128.  status: iris::StatusBlock on the device or null.
// Returns 0, or a negative code with a message in iris_attention_last_error().
int iris_k_attention_fwd(const void* qkv, int64_t ld_qkv, void* out, int64_t ldo, int batch, int seq, int heads,
                         int causal, int dtype, void* status, uint64_t timeout_ns, void* stream) {
  using namespace iris::attn;
  g_attn_err[0] = 0;
  if (!qkv || !out || batch < 1 || heads < 1 || seq < BQ || seq % BQ != 0) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: need buffers, batch, heads >= 1 and seq a multiple of %d", BQ);
    return -1;
  }
  if (reinterpret_cast<uintptr_t>(qkv) % 16 || reinterpret_cast<uintptr_t>(out) % 16 || (ld_qkv * 2) % 16 ||
      (ldo * 2) % 16 || ld_qkv < 3ll * heads * D || ldo < (int64_t)heads * D) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: 16-byte aligned buffers and pitches of at least the row");
    return -1;
  }
  if (dtype != 0 && dtype != 1) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: dtype must be 0 (bf16) or 1 (fp16)");
    return -1;
  }
  EncodeTiledFn enc = attn_encode_fn();
  if (!enc) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: cuTensorMapEncodeTiled is not available");
    return -2;
  }
  Params p;
  memset(&p, 0, sizeof(p));
  cuuint64_t dims[2] = {(cuuint64_t)3 * heads * D, (cuuint64_t)batch * seq};
  cuuint64_t strides[1] = {(cuuint64_t)ld_qkv * 2};
  cuuint32_t box[2] = {64, 128};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = enc(&p.tm, dtype ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2,
                   const_cast<void*>(qkv), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: cuTensorMapEncodeTiled failed with %d", (int)r);
    return -2;
  }
  p.out = out;
  p.ldo = ldo;
  p.status = static_cast<iris::StatusBlock*>(status);
  p.timeout_ns = timeout_ns ? timeout_ns : 2000000000ull;
  p.batch = batch;
  p.seq = seq;
  p.heads = heads;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = 1.4426950408889634f / 11.313708498984761f;   // log2(e) / sqrt(128)
  auto kern = dtype ? attention_fwd_kernel<true> : attention_fwd_kernel<false>;
  static std::once_flag attr_once[2];
  cudaError_t e = cudaSuccess;
  std::call_once(attr_once[dtype], [&]() {
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBytes);
  });
  if (e != cudaSuccess) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    return -3;
  }
  const int grid = batch * heads * (seq / BQ);
  kern<<<grid, kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(p);
  e = cudaGetLastError();
  if (e != cudaSuccess) {
    snprintf(g_attn_err, sizeof(g_attn_err), "attention: launch: %s", cudaGetErrorString(e));
    return -3;
  }
  return 0;
}

}  // extern "C"
