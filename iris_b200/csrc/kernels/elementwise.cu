// elementwise.cu — the memory-bound pieces of the tensor-parallel decoder block: RMSNorm, residual add fused with
// the RMSNorm that follows it, SwiGLU and the plain residual add, bf16 in / bf16 out with fp32 arithmetic, 16-byte
// vector accesses.
//
// No counterpart in the reference (it has no model code); they exist for the tensor-parallel block built on
// the fused GEMM + collective kernels.  RMSNorm writes straight into the row block that the all-gather -> GEMM
// kernel pushes to the peers, so the normalised activations are never copied.
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace {

__device__ __forceinline__ void unpack8(uint4 v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 o;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return o;
}

// One CTA per row; cols % 8 == 0.  out[r, :] = x[r, :] * rsqrt(mean(x^2) + eps) * w
template <int kThreads>
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                           const __nv_bfloat16* __restrict__ w,
                                                           __nv_bfloat16* __restrict__ out, int64_t ldo, int cols,
                                                           float eps) {
  __shared__ float red[kThreads / 32];
  const int r = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)r * ldx);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)r * ldo);
  const int nv = cols / 8;
  float ss = 0.f;
  for (int i = threadIdx.x; i < nv; i += kThreads) {
    float f[8];
    unpack8(xr[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) tot += red[i];
  const float scale = rsqrtf(tot / (float)cols + eps);
  for (int i = threadIdx.x; i < nv; i += kThreads) {
    float f[8], g[8];
    unpack8(xr[i], f);  // second read hits L1/L2
    unpack8(wv[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = f[j] * scale * g[j];
    orow[i] = pack8(f);
  }
}

// As above for rows of at most kThreads * VPT vectors: the row stays in registers between the two passes, so x is
// read once (the generic kernel's second read hits L2 but costs a second round of load latency per row).
template <int kThreads, int VPT>
__global__ void __launch_bounds__(kThreads) rmsnorm_reg_kernel(const __nv_bfloat16* __restrict__ x, int64_t ldx,
                                                               const __nv_bfloat16* __restrict__ w,
                                                               __nv_bfloat16* __restrict__ out, int64_t ldo, int cols,
                                                               float eps) {
  __shared__ float red[kThreads / 32];
  const int r = blockIdx.x;
  const uint4* xr = reinterpret_cast<const uint4*>(x + (int64_t)r * ldx);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)r * ldo);
  const int nv = cols / 8;
  uint4 xv[VPT], wr[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * kThreads;
    if (i < nv) {
      xv[v] = xr[i];
      wr[v] = wv[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    if (threadIdx.x + v * kThreads < nv) {
      float f[8];
      unpack8(xv[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) tot += red[i];
  const float scale = rsqrtf(tot / (float)cols + eps);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * kThreads;
    if (i < nv) {
      float f[8], g[8];
      unpack8(xv[v], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * scale * g[j];
      orow[i] = pack8(f);
    }
  }
}

// Residual add fused with the norm that follows it: x[r, :] += y[r, :] (stored back, the residual stream), then
// out[r, :] = x[r, :] * rsqrt(mean(x^2) + eps) * w.  The row stays in registers: x and y are read once, x and out
// written once, instead of the three reads and two writes of the two separate kernels.  Rows of at most
// kThreads * VPT vectors.
template <int kThreads, int VPT>
__global__ void __launch_bounds__(kThreads) add_rmsnorm_reg_kernel(__nv_bfloat16* __restrict__ x, int64_t ldx,
                                                                   const __nv_bfloat16* __restrict__ y, int64_t ldy,
                                                                   const __nv_bfloat16* __restrict__ w,
                                                                   __nv_bfloat16* __restrict__ out, int64_t ldo,
                                                                   int cols, float eps) {
  __shared__ float red[kThreads / 32];
  const int r = blockIdx.x;
  uint4* xr = reinterpret_cast<uint4*>(x + (int64_t)r * ldx);
  const uint4* yr = reinterpret_cast<const uint4*>(y + (int64_t)r * ldy);
  const uint4* wv = reinterpret_cast<const uint4*>(w);
  uint4* orow = reinterpret_cast<uint4*>(out + (int64_t)r * ldo);
  const int nv = cols / 8;
  uint4 xv[VPT], yv[VPT], wr[VPT];
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * kThreads;
    if (i < nv) {
      xv[v] = xr[i];
      yv[v] = yr[i];
      wr[v] = wv[i];
    }
  }
  float ss = 0.f;
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * kThreads;
    if (i < nv) {
      float f[8], g[8];
      unpack8(xv[v], f);
      unpack8(yv[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] += g[j];
      xv[v] = pack8(f);        // the residual stream is bf16: the norm sees the rounded sum, as the unfused pair does
      xr[i] = xv[v];
      unpack8(xv[v], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < kThreads / 32; ++i) tot += red[i];
  const float scale = rsqrtf(tot / (float)cols + eps);
#pragma unroll
  for (int v = 0; v < VPT; ++v) {
    const int i = threadIdx.x + v * kThreads;
    if (i < nv) {
      float f[8], g[8];
      unpack8(xv[v], f);
      unpack8(wr[v], g);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = f[j] * scale * g[j];
      orow[i] = pack8(f);
    }
  }
}

// silu(a) * b with two special-function operations per element (ex2 and rcp) and no IEEE division: the kernel has
// to stay below about 25 instructions per element to be bound by memory rather than by instruction issue.
__device__ __forceinline__ float silu_mul(float a, float b) {
  return __fdividef(a, 1.f + __expf(-a)) * b;
}

// out[r, c] = silu(gu[r, c]) * gu[r, inter + c]; four independent 16-byte load pairs in flight per thread.
// Index: 32-bit (fewer instructions than 64-bit division) unless the matrix has 2^31 vectors or more.
template <class Index>
__global__ void __launch_bounds__(256) swiglu_kernel(const __nv_bfloat16* __restrict__ gu, int64_t ldg,
                                                     __nv_bfloat16* __restrict__ out, int64_t ldo, int rows, int inter) {
  constexpr int U = 4;
  const Index nv = (Index)(inter / 8);
  const Index total = (Index)rows * nv;
  const Index stride = (Index)gridDim.x * blockDim.x;
  for (Index i0 = (Index)blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += U * stride) {
    uint4 g[U], u[U];
    int64_t oo[U];
#pragma unroll
    for (int q = 0; q < U; ++q) {
      const Index i = i0 + q * stride;
      if (i < total) {
        const Index r = i / nv;
        const Index c = i - r * nv;
        const __nv_bfloat16* src = gu + (int64_t)r * ldg + (int64_t)c * 8;
        g[q] = *reinterpret_cast<const uint4*>(src);
        u[q] = *reinterpret_cast<const uint4*>(src + inter);
        oo[q] = (int64_t)r * ldo + (int64_t)c * 8;
      }
    }
#pragma unroll
    for (int q = 0; q < U; ++q) {
      if (i0 + q * stride < total) {
        float a[8], b[8];
        unpack8(g[q], a);
        unpack8(u[q], b);
#pragma unroll
        for (int j = 0; j < 8; ++j) a[j] = silu_mul(a[j], b[j]);
        *reinterpret_cast<uint4*>(out + oo[q]) = pack8(a);
      }
    }
  }
}

// x[r, :] += y[r, :]
__global__ void residual_add_kernel(__nv_bfloat16* __restrict__ x, int64_t ldx, const __nv_bfloat16* __restrict__ y,
                                    int64_t ldy, int rows, int cols) {
  const int nv = cols / 8;
  const int64_t total = (int64_t)rows * nv;
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
    const int r = (int)(i / nv), c = (int)(i - (int64_t)r * nv);
    uint4* xp = reinterpret_cast<uint4*>(x + (int64_t)r * ldx + c * 8);
    float a[8], b[8];
    unpack8(*xp, a);
    unpack8(*reinterpret_cast<const uint4*>(y + (int64_t)r * ldy + c * 8), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] += b[j];
    *xp = pack8(a);
  }
}

int grid_for(int64_t work_items, int block) {
  int64_t g = (work_items + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > 148 * 8 ? 148 * 8 : g));
}

}  // namespace

extern "C" {

int iris_k_rmsnorm_bf16(const void* x, int64_t ldx, const void* w, void* out, int64_t ldo, int rows, int cols,
                        float eps, void* stream) {
  if (cols % 8 != 0 || rows < 1) return -2;
  const __nv_bfloat16* xp = (const __nv_bfloat16*)x;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  __nv_bfloat16* op = (__nv_bfloat16*)out;
  cudaStream_t st = (cudaStream_t)stream;
  const int nv = cols / 8;
  if (nv <= 256) rmsnorm_reg_kernel<256, 1><<<rows, 256, 0, st>>>(xp, ldx, wp, op, ldo, cols, eps);
  else if (nv <= 512) rmsnorm_reg_kernel<256, 2><<<rows, 256, 0, st>>>(xp, ldx, wp, op, ldo, cols, eps);
  else if (nv <= 1024) rmsnorm_reg_kernel<256, 4><<<rows, 256, 0, st>>>(xp, ldx, wp, op, ldo, cols, eps);
  else rmsnorm_kernel<256><<<rows, 256, 0, st>>>(xp, ldx, wp, op, ldo, cols, eps);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
// x += y; out = rmsnorm(x) * w.  Returns -3 when the row is too long for the register-resident kernel (the caller
// then runs the two separate kernels).
int iris_k_add_rmsnorm_bf16(void* x, int64_t ldx, const void* y, int64_t ldy, const void* w, void* out, int64_t ldo,
                            int rows, int cols, float eps, void* stream) {
  if (cols % 8 != 0 || rows < 1) return -2;
  __nv_bfloat16* xp = (__nv_bfloat16*)x;
  const __nv_bfloat16* yp = (const __nv_bfloat16*)y;
  const __nv_bfloat16* wp = (const __nv_bfloat16*)w;
  __nv_bfloat16* op = (__nv_bfloat16*)out;
  cudaStream_t st = (cudaStream_t)stream;
  const int nv = cols / 8;
  if (nv <= 256) add_rmsnorm_reg_kernel<256, 1><<<rows, 256, 0, st>>>(xp, ldx, yp, ldy, wp, op, ldo, cols, eps);
  else if (nv <= 512) add_rmsnorm_reg_kernel<256, 2><<<rows, 256, 0, st>>>(xp, ldx, yp, ldy, wp, op, ldo, cols, eps);
  else if (nv <= 1024) add_rmsnorm_reg_kernel<256, 4><<<rows, 256, 0, st>>>(xp, ldx, yp, ldy, wp, op, ldo, cols, eps);
  else return -3;
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int iris_k_swiglu_bf16(const void* gu, int64_t ldg, void* out, int64_t ldo, int rows, int inter, void* stream) {
  if (inter % 8 != 0 || rows < 1) return -2;
  const int64_t vecs = (int64_t)rows * (inter / 8);
  const int grid = grid_for((vecs + 3) / 4, 256);
  if (vecs + 4ll * grid * 256 < (1ll << 32))
    swiglu_kernel<uint32_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, ldg, (__nv_bfloat16*)out,
                                                                     ldo, rows, inter);
  else
    swiglu_kernel<int64_t><<<grid, 256, 0, (cudaStream_t)stream>>>((const __nv_bfloat16*)gu, ldg, (__nv_bfloat16*)out,
                                                                    ldo, rows, inter);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}
int iris_k_residual_add_bf16(void* x, int64_t ldx, const void* y, int64_t ldy, int rows, int cols, void* stream) {
  if (cols % 8 != 0 || rows < 1) return -2;
  residual_add_kernel<<<grid_for((int64_t)rows * cols / 8, 256), 256, 0, (cudaStream_t)stream>>>(
      (__nv_bfloat16*)x, ldx, (const __nv_bfloat16*)y, ldy, rows, cols);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
