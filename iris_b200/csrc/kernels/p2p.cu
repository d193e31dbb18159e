// p2p.cu — point-to-point and all-peer RMA bandwidth kernels, the int32 fill kernel and the
// producer/consumer message-passing kernels.
//
// Reference kernels and what replaces them here:
//   examples/00_load/load_bench.py:20-61              -> p2p_load   (remote read -> local write) + local_store
//   examples/01_store/store_bench.py:20-46            -> p2p_store  (write the word index into the peer)
//   examples/02_all_load/all_load_bench.py:41-86      -> p2p_all_load  (sum of the same slice of every rank)
//   examples/03_all_store/all_store_bench.py:21-49    -> p2p_all_store (write to every other rank)
//   examples/04_atomic_add/atomic_add_bench.py:20-41  -> p2p_atomic_add (relaxed, system scope, result unused)
//   examples/05_atomic_xchg/atomic_xchg_bench.py:20-44-> p2p_atomic_xchg (old values stored locally)
//   examples/06_message_passing/*.py                  -> mp_kernel (chunk copy + release flag / acquire wait)
//   iris/util.py:107-128                              -> memset_i32
// The reference launches one 512-element program per block of data; here each kernel is a persistent
// grid-stride loop over 16-byte vectors with several accesses in flight per thread, which is what NVLink
// needs to reach its bandwidth.
#include <cuda_runtime.h>

#include "iris/iris.cuh"

using namespace iris;

namespace {

constexpr int kUnroll = 8;

__device__ __forceinline__ uint4 index_pattern(size_t vec_index) {
  const uint32_t w = (uint32_t)(vec_index * 4);
  return make_uint4(w, w + 1, w + 2, w + 3);
}

// dst_local[i] = remote(src)[i]
__global__ void p2p_load_kernel(const uint4* src_sym, uint4* dst_local, size_t n16, int cur, int tgt,
                                const uint64_t* hb) {
  const uint4* src = translate(src_sym, cur, tgt, hb);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  for (; i + (kUnroll - 1) * stride < n16; i += kUnroll * stride) {
    uint4 v[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) v[u] = ld_v4_stream(src + i + u * stride);
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) st_v4(dst_local + i + u * stride, v[u]);
  }
  for (; i < n16; i += stride) st_v4(dst_local + i, ld_v4_stream(src + i));
}

// remote(dst)[w] = w for every 32-bit word w (the reference stores the element index).
__global__ void p2p_store_kernel(uint4* dst_sym, size_t n16, int cur, int tgt, const uint64_t* hb) {
  uint4* dst = translate(dst_sym, cur, tgt, hb);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) st_v4(dst + i, index_pattern(i));
}

template <class T>
struct Vec16;
template <>
struct Vec16<float> {
  static __device__ __forceinline__ void add(float* acc, uint4 v) {
    acc[0] += __uint_as_float(v.x);
    acc[1] += __uint_as_float(v.y);
    acc[2] += __uint_as_float(v.z);
    acc[3] += __uint_as_float(v.w);
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    return make_uint4(__float_as_uint(acc[0]), __float_as_uint(acc[1]), __float_as_uint(acc[2]),
                      __float_as_uint(acc[3]));
  }
  static constexpr int kAcc = 4;
};
template <>
struct Vec16<__half> {
  static __device__ __forceinline__ void add(float* acc, uint4 v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __half22float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    uint4 o;
    __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    return o;
  }
  static constexpr int kAcc = 8;
};
template <>
struct Vec16<__nv_bfloat16> {
  static __device__ __forceinline__ void add(float* acc, uint4 v) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      acc[2 * i] += f.x;
      acc[2 * i + 1] += f.y;
    }
  }
  static __device__ __forceinline__ uint4 pack(const float* acc) {
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(acc[2 * i], acc[2 * i + 1]);
    return o;
  }
  static constexpr int kAcc = 8;
};

// out_local[i] = sum over the first `active` (<= 8) ranks of remote_r(src)[i].
template <class T>
__global__ void p2p_all_load_kernel(const uint4* src_sym, uint4* out_local, size_t n16, int cur, int active,
                                    const uint64_t* hb) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    uint4 v[8];
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < active) v[r] = ld_v4_stream(translate(src_sym, cur, (cur + r) % active, hb) + i);
    float acc[Vec16<T>::kAcc] = {};
#pragma unroll
    for (int r = 0; r < 8; ++r)
      if (r < active) Vec16<T>::add(acc, v[r]);
    st_v4(out_local + i, Vec16<T>::pack(acc));
  }
}

// remote_r(dst)[w] = w for every OTHER rank r.
__global__ void p2p_all_store_kernel(uint4* dst_sym, size_t n16, int cur, int active, const uint64_t* hb) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint4 v = index_pattern(i);
    for (int r = 1; r < active; ++r) st_v4(translate(dst_sym, cur, (cur + r) % active, hb) + i, v);
  }
}

// remote(buf)[i] += 1.0f, relaxed, system scope, result discarded.
__global__ void p2p_atomic_add_f32_kernel(float* buf_sym, size_t n, int cur, int tgt, const uint64_t* hb, int vec4) {
  float* buf = translate(buf_sym, cur, tgt, hb);
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  if (vec4) {
    const size_t n4 = n / 4;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride)
      red_add_v4_f32(buf + 4 * i, 1.f, 1.f, 1.f, 1.f);
    for (size_t i = n4 * 4 + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) red_add_f32(buf + i, 1.f);
  } else {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) red_add_f32(buf + i, 1.f);
  }
}

// The same for the other element types the device API adds in hardware (fp16, bf16, int32, int64): one relaxed,
// system-scope reduction per element (examples/04_atomic_add/atomic_add_bench.py:20-41 of the reference).
template <class T>
__global__ void p2p_atomic_add_kernel(T* buf_sym, size_t n, int cur, int tgt, const uint64_t* hb, T one) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    atomic_add<Sem::relaxed, Scope::sys>(buf_sym + i, one, cur, tgt, hb);
}

// out_local[i] = atomic_xchg(remote(buf)[i], 1), relaxed, system scope.
__global__ void p2p_atomic_xchg_i32_kernel(int* buf_sym, int* out_local, size_t n, int cur, int tgt,
                                           const uint64_t* hb) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
    out_local[i] = atomic_xchg<Sem::relaxed, Scope::sys>(buf_sym + i, 1, cur, tgt, hb);
}

__global__ void local_store_kernel(uint4* dst, size_t n16) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) st_v4(dst + i, index_pattern(i));
}

__global__ void memset_i32_kernel(int* p, int value, size_t n) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) p[i] = value;
}

// ---- message passing -----------------------------------------------------------------------------
struct MpArgs {
  const uint64_t* hb;
  uint64_t src_off;     // producer's source buffer (symmetric offset)
  uint64_t dst_off;     // consumer's landing buffer
  uint64_t out_off;     // consumer's result buffer: 2 * landed value (fp32)
  uint64_t flags_off;   // uint32 per chunk, in the consumer's heap
  uint64_t status_off;  // StatusBlock in each rank's heap
  uint64_t chunk_bytes; // multiple of 16
  uint64_t timeout_ns;
  int nchunks;
  int producer, consumer;
  int roles;            // bit 0: this launch runs the producer blocks, bit 1: the consumer blocks
  int use_put;          // 1: block-cooperative put; 0: per-thread load + store of floats
  uint32_t epoch;       // flag value that marks "chunk of this call has landed"; 0: both sides count their calls in
                        // device memory (word [nchunks] of arrive / flags: calls completed, word [nchunks + 1]:
                        // blocks of the running launch that have left), so that a launch has no per-call argument
                        // and can be replayed from a CUDA graph
  int parts;            // blocks per chunk: every chunk is cut into `parts` slices of whole 16-byte vectors
  uint64_t arrive_off;  // uint32 per chunk, in the producer's heap: slices of the chunk copied so far (back at 0
                        // when the chunk's flag has been raised)
  int blocks;           // blocks per role: block b handles the (chunk, slice) pairs b, b + blocks, ... in that order
};

// Blocks [0, blocks) produce (when roles & 1); the following `blocks` blocks consume (when roles & 2).
// A chunk is cut into `parts` slices, so that one chunk is moved by `parts` SMs at once and a hand-off of a few large
// chunks still uses the whole GPU.  Block b of a role handles the (chunk, slice) pairs b, b + blocks, ... in order:
// with blocks = nchunks * parts all chunks travel at once and land together at the end; with fewer blocks the chunks
// complete one group after the other, and the consumer works on the early ones while the later ones are on the link.
// Producer: copy the slice into the consumer's buffer, make it visible (barrier + one system-scope fence), count it on
// the chunk's arrival counter; the block that completes the count raises the CONSUMER's flag with release semantics
// and puts the counter back to zero.  Consumer: every block of the chunk waits (bounded, acquire) on the chunk's flag
// in its own memory, then writes out = 2 * landed for its slice.
__global__ void mp_kernel(MpArgs a) {
  __shared__ uint32_t verdict, epoch_s;
  int b = blockIdx.x;
  const int nblk = a.nchunks * a.parts;
  const int R = a.blocks;
  const bool has_prod = a.roles & 1;
  const bool producing = has_prod && b < R;
  // this side's call counter: the producer's next to its arrival counters, the consumer's next to its flags
  const uint64_t counters = producing ? a.hb[a.producer] + a.arrive_off : a.hb[a.consumer] + a.flags_off;
  uint32_t* calls = reinterpret_cast<uint32_t*>(counters) + a.nchunks;
  if (threadIdx.x == 0) epoch_s = a.epoch ? a.epoch : *reinterpret_cast<volatile uint32_t*>(calls) + 1u;
  __syncthreads();
  const uint32_t epoch = epoch_s;
  // the last block of a side to leave advances that side's counter (nothing to do with a host-given epoch)
  auto leave = [&]() {
    if (a.epoch == 0 && threadIdx.x == 0 && atomicAdd(calls + 1, 1u) + 1u == (uint32_t)R) {
      *reinterpret_cast<volatile uint32_t*>(calls + 1) = 0u;
      *reinterpret_cast<volatile uint32_t*>(calls) = epoch;
    }
  };
  // slice q of a chunk: whole 16-byte vectors, the last slice takes the remainder
  const uint64_t vecs = a.chunk_bytes / 16;
  const uint64_t per = (vecs + a.parts - 1) / a.parts;
  if (has_prod && b < R) {
    for (int w = b; w < nblk; w += R) {
      const int c = w / a.parts, q = w - c * a.parts;
      const uint64_t v0 = per * q < vecs ? per * q : vecs, v1 = v0 + per < vecs ? v0 + per : vecs;
      const uint64_t off = (uint64_t)c * a.chunk_bytes + v0 * 16, bytes = (v1 - v0) * 16;
      const uint64_t base = a.hb[a.producer];
      const char* src = reinterpret_cast<const char*>(base + a.src_off) + off;
      char* dst_sym = reinterpret_cast<char*>(base + a.dst_off) + off;
      if (a.use_put) {
        put_block(src, dst_sym, bytes, a.producer, a.consumer, a.hb);
      } else {
        const float* s = reinterpret_cast<const float*>(src);
        float* d = reinterpret_cast<float*>(dst_sym);
        for (size_t i = threadIdx.x; i < bytes / 4; i += blockDim.x)
          store(d + i, load(s + i, a.producer, a.producer, a.hb), a.producer, a.consumer, a.hb);
      }
      // One thread publishes for the block: the barrier orders every thread's stores before its system-scope fence
      // (fences are cumulative), and only its warp waits for the link round trip; the others start the next slice.
      __syncthreads();
      if (threadIdx.x == 0) {
        fence_sys();
        uint32_t* cnt = reinterpret_cast<uint32_t*>(base + a.arrive_off) + c;
        const uint32_t old = atomic_add<Sem::acq_rel, Scope::gpu>(cnt, 1u, 0, 0, a.hb);
        if (old + 1 == (uint32_t)a.parts) {
          *cnt = 0;  // every slice has arrived: nobody touches the counter again in this call
          uint32_t* flag = reinterpret_cast<uint32_t*>(base + a.flags_off) + c;
          signal_set(flag, epoch, a.producer, a.consumer, a.hb);
        }
      }
    }
    leave();
    return;
  }
  if (has_prod) b -= R;
  if (!(a.roles & 2) || b >= R) return;
  for (int w = b; w < nblk; w += R) {
    const int c = w / a.parts, q = w - c * a.parts;
    const uint64_t v0 = per * q < vecs ? per * q : vecs, v1 = v0 + per < vecs ? v0 + per : vecs;
    const uint64_t base = a.hb[a.consumer];
    if (threadIdx.x == 0) {
      const uint32_t* flag = reinterpret_cast<const uint32_t*>(base + a.flags_off) + c;
      verdict = wait_until_ge(flag, epoch, a.timeout_ns, reinterpret_cast<StatusBlock*>(base + a.status_off),
                              /*where=*/60, (uint32_t)a.consumer, (uint32_t)c);
    }
    __syncthreads();
    if (verdict != kOk) {  // uniform over the block
      leave();
      return;
    }
    const float4* in = reinterpret_cast<const float4*>(base + a.dst_off + (uint64_t)c * a.chunk_bytes);
    float4* out = reinterpret_cast<float4*>(base + a.out_off + (uint64_t)c * a.chunk_bytes);
    for (size_t i = v0 + threadIdx.x; i < v1; i += blockDim.x) {
      float4 v = in[i];
      out[i] = make_float4(2.f * v.x, 2.f * v.y, 2.f * v.z, 2.f * v.w);
    }
    __syncthreads();  // everybody has read `verdict` before thread 0 writes the next one
  }
  leave();
}

// Device-side barrier across ranks: one thread adds 1 to counter[0] of every rank (release, system scope),
// then waits (bounded) until its own counter reaches calls * world.  Streams of different GPUs are
// aligned to within a few microseconds when this kernel completes.  The number of calls so far is kept in
// counter[1] of the rank's own heap and advanced by the kernel, so that a launch has no per-call argument and can
// be replayed from a CUDA graph.
__global__ void device_barrier_kernel(const uint64_t* hb, uint64_t counter_off, uint64_t status_off, int rank,
                                      int world, uint64_t timeout_ns) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  volatile uint32_t* calls = reinterpret_cast<volatile uint32_t*>(hb[rank] + counter_off) + 1;
  const uint32_t call = *calls + 1u;
  const uint32_t target = call * (uint32_t)world;
  fence_sys();  // one fence, then relaxed arrivals: a release per rank would wait for the previous rank's answer
  for (int i = 0; i < world; ++i) {
    const int t = (rank + 1 + i) % world;
    red_relaxed_sys_add(reinterpret_cast<uint32_t*>(hb[t] + counter_off), 1u);
  }
  wait_until_ge(reinterpret_cast<const uint32_t*>(hb[rank] + counter_off), target, timeout_ns,
                reinterpret_cast<StatusBlock*>(hb[rank] + status_off), /*where=*/70, (uint32_t)rank, target);
  *calls = call;
}

int check_launch() { return cudaGetLastError() == cudaSuccess ? 0 : -1; }

}  // namespace

extern "C" {

int iris_k_p2p_load(const void* src_sym, void* dst_local, uint64_t bytes, int cur, int tgt, const uint64_t* hb,
                    int grid, int block, void* stream) {
  p2p_load_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((const uint4*)src_sym, (uint4*)dst_local, bytes / 16, cur,
                                                            tgt, hb);
  return check_launch();
}
int iris_k_p2p_store(void* dst_sym, uint64_t bytes, int cur, int tgt, const uint64_t* hb, int grid, int block,
                     void* stream) {
  p2p_store_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((uint4*)dst_sym, bytes / 16, cur, tgt, hb);
  return check_launch();
}
int iris_k_local_store(void* dst, uint64_t bytes, int grid, int block, void* stream) {
  local_store_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((uint4*)dst, bytes / 16);
  return check_launch();
}
// dtype: 4 = fp16, 5 = bf16, 6 = fp32 (iris::ops::DType numbering)
int iris_k_p2p_all_load(const void* src_sym, void* out_local, uint64_t bytes, int dtype, int cur, int active,
                        const uint64_t* hb, int grid, int block, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  const size_t n16 = bytes / 16;
  if (active < 1 || active > 8) return -3;
  if (dtype == 6) p2p_all_load_kernel<float><<<grid, block, 0, st>>>((const uint4*)src_sym, (uint4*)out_local, n16, cur, active, hb);
  else if (dtype == 4) p2p_all_load_kernel<__half><<<grid, block, 0, st>>>((const uint4*)src_sym, (uint4*)out_local, n16, cur, active, hb);
  else if (dtype == 5) p2p_all_load_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const uint4*)src_sym, (uint4*)out_local, n16, cur, active, hb);
  else return -2;
  return check_launch();
}
int iris_k_p2p_all_store(void* dst_sym, uint64_t bytes, int cur, int active, const uint64_t* hb, int grid, int block,
                         void* stream) {
  p2p_all_store_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((uint4*)dst_sym, bytes / 16, cur, active, hb);
  return check_launch();
}
int iris_k_p2p_atomic_add_f32(void* buf_sym, uint64_t n, int cur, int tgt, const uint64_t* hb, int vec4, int grid,
                              int block, void* stream) {
  p2p_atomic_add_f32_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((float*)buf_sym, n, cur, tgt, hb, vec4);
  return check_launch();
}
// dtype: iris::ops::DType numbering (2 = int32, 3 = int64, 4 = fp16, 5 = bf16, 6 = fp32)
int iris_k_p2p_atomic_add(void* buf_sym, uint64_t n, int dtype, int cur, int tgt, const uint64_t* hb, int grid,
                          int block, void* stream) {
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == 6) p2p_atomic_add_f32_kernel<<<grid, block, 0, st>>>((float*)buf_sym, n, cur, tgt, hb, 0);
  else if (dtype == 4) p2p_atomic_add_kernel<__half><<<grid, block, 0, st>>>((__half*)buf_sym, n, cur, tgt, hb, __float2half(1.f));
  else if (dtype == 5) p2p_atomic_add_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((__nv_bfloat16*)buf_sym, n, cur, tgt, hb, __float2bfloat16(1.f));
  else if (dtype == 2) p2p_atomic_add_kernel<int><<<grid, block, 0, st>>>((int*)buf_sym, n, cur, tgt, hb, 1);
  else if (dtype == 3) p2p_atomic_add_kernel<long long><<<grid, block, 0, st>>>((long long*)buf_sym, n, cur, tgt, hb, 1ll);
  else return -2;
  return check_launch();
}
int iris_k_p2p_atomic_xchg_i32(void* buf_sym, void* out_local, uint64_t n, int cur, int tgt, const uint64_t* hb,
                               int grid, int block, void* stream) {
  p2p_atomic_xchg_i32_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((int*)buf_sym, (int*)out_local, n, cur, tgt, hb);
  return check_launch();
}
int iris_k_memset_i32(void* p, int value, uint64_t n, void* stream) {
  if (n == 0) return 0;
  const int block = 256;
  const int grid = (int)((n + block - 1) / block < 1184 ? (n + block - 1) / block : 1184);
  memset_i32_kernel<<<grid, block, 0, (cudaStream_t)stream>>>((int*)p, value, n);
  return check_launch();
}

int iris_k_device_barrier(const uint64_t* hb, uint64_t counter_off, uint64_t status_off, int rank, int world,
                          uint64_t timeout_ns, void* stream) {
  device_barrier_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(hb, counter_off, status_off, rank, world, timeout_ns);
  return check_launch();
}

// roles: 1 producer side only, 2 consumer side only, 3 both in one (cooperative) launch on one GPU.
// parts: slices per chunk (>= 1); blocks: thread blocks per role (0 or more than nchunks * parts: one per slice);
// arrive_off: uint32[nchunks] in the producer's heap, zero before the first call.
int iris_k_message_passing(const uint64_t* hb, uint64_t src_off, uint64_t dst_off, uint64_t out_off,
                           uint64_t flags_off, uint64_t status_off, uint64_t chunk_bytes, int nchunks, int producer,
                           int consumer, int roles, int use_put, uint32_t epoch, uint64_t timeout_ns, int block,
                           int parts, uint64_t arrive_off, int blocks, void* stream) {
  if (chunk_bytes % 16 != 0 || nchunks < 1 || parts < 1) return -2;
  if (roles == 3) {
    // Producer and consumer blocks wait on one another: all of them must be resident at once.  Lower `parts` to
    // what the device holds (both sides of one launch use the same value, so the arrival counts stay consistent).
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess ||
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, mp_kernel, block, 0) != cudaSuccess)
      return -3;
    const int fit = (sms * per_sm) / 2;   // blocks per role that are resident together with the other role's
    if (fit < 1) return -4;
    if (blocks <= 0 || blocks > fit) blocks = fit;
  }
  if (blocks <= 0 || blocks > nchunks * parts) blocks = nchunks * parts;
  MpArgs a{hb, src_off, dst_off, out_off, flags_off, status_off, chunk_bytes, timeout_ns, nchunks, producer, consumer,
           roles, use_put, epoch, parts, arrive_off, blocks};
  const int grid = (roles == 3 ? 2 : 1) * blocks;
  cudaError_t e;
  if (roles == 3) {
    // Producer and consumer blocks wait on one another: they must be co-resident.
    void* args[] = {&a};
    e = cudaLaunchCooperativeKernel((void*)mp_kernel, dim3(grid), dim3(block), args, 0, (cudaStream_t)stream);
  } else {
    mp_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(a);
    e = cudaGetLastError();
  }
  return e == cudaSuccess ? 0 : -1;
}

}  // extern "C"
