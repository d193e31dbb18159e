// nvls.cu — collectives that let the NVLink switch do the work (multimem instructions on the heap's multicast
// mapping; see include/iris/nvls.cuh).  They need a context created with heap_mode="vmm" and IRIS_NVLS=1.
//
//   nvls_all_store   every 16-byte vector is stored ONCE and lands in all ranks (the NVLS form of
//                    examples/03_all_store/all_store_bench.py:21-49 of the reference)
//   nvls_all_reduce  in-place sum of a bf16 buffer over all ranks: rank r reduces slice r with
//                    multimem.ld_reduce (the switch adds the W copies) and broadcasts the result with
//                    multimem.st, then a device-side barrier (the library-free form of the reference's
//                    all-reduce baseline, examples/benchmark/reference/all_reduce.py:128)
#include <cuda_runtime.h>

#include "iris/nvls.cuh"

using namespace iris;

namespace {

__global__ void nvls_all_store_kernel(uint64_t mc_ptr, size_t n16) {
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += stride) {
    const uint32_t w = (uint32_t)(i * 4);
    nvls::st_v4(reinterpret_cast<void*>(mc_ptr + i * 16), make_uint4(w, w + 1, w + 2, w + 3));
  }
}

// counter: uint32[3] at symmetric offset counter_off.  [0]: arrivals, cumulative over calls, written by every rank
// through the multicast address; two barrier phases per call, every block of every rank arrives once per phase.
// [1] (local): arrivals counted up to the end of the previous call; [2] (local): blocks of this launch that have left.
// The last block to leave advances [1] and clears [2], so a launch has no per-call argument and can be replayed from
// a CUDA graph, with any grid size (the same on every rank) from call to call.
__device__ __forceinline__ void all_reduce_leave(uint32_t* my_counter, uint32_t base, int world) {
  if (atomicAdd(my_counter + 2, 1u) + 1u == gridDim.x) {
    *reinterpret_cast<volatile uint32_t*>(my_counter + 2) = 0u;
    *reinterpret_cast<volatile uint32_t*>(my_counter + 1) = base + 2u * gridDim.x * (uint32_t)world;
  }
}

__global__ void nvls_all_reduce_bf16_kernel(uint64_t mc_buf, const uint64_t* hb, uint64_t counter_off,
                                            uint64_t status_off, size_t n16, int rank, int world,
                                            uint64_t timeout_ns, uint64_t mc_base) {
  __shared__ uint32_t ok, base_s;
  const size_t per = (n16 + world - 1) / world;
  const size_t lo = per * rank, hi = lo + per < n16 ? lo + per : n16;
  uint32_t* my_counter = reinterpret_cast<uint32_t*>(hb[rank] + counter_off);
  if (threadIdx.x == 0) base_s = *reinterpret_cast<volatile uint32_t*>(my_counter + 1);
  // Phase 0: every rank's input is complete (kernel ordering on its own stream) -> all blocks of all ranks arrive.
  __syncthreads();
  const uint32_t base = base_s;
  const uint32_t target0 = base + (uint32_t)(gridDim.x * world);
  if (threadIdx.x == 0) {
    fence_sys();
    nvls::red_release_add_u32(reinterpret_cast<void*>(mc_base + counter_off), 1u);
    ok = wait_until_ge(my_counter, target0, timeout_ns, reinterpret_cast<StatusBlock*>(hb[rank] + status_off), 80,
                       (uint32_t)rank, 0) == kOk;
  }
  __syncthreads();
  if (!ok) {
    // Phase 0 timed out: no data is touched, but the phase-1 arrival is still made, so that this rank keeps adding
    // exactly two arrivals per block and call to every rank's counter (the invariant the host's targets rest on).
    if (threadIdx.x == 0) {
      nvls::red_release_add_u32(reinterpret_cast<void*>(mc_base + counter_off), 1u);
      all_reduce_leave(my_counter, base, world);
    }
    return;
  }
  const size_t stride = (size_t)gridDim.x * blockDim.x;
  for (size_t i = lo + (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < hi; i += stride) {
    const uint4 v = nvls::ld_reduce_add_bf16x8(reinterpret_cast<const void*>(mc_buf + i * 16));
    nvls::st_v4(reinterpret_cast<void*>(mc_buf + i * 16), v);
  }
  // Phase 1: results of every rank's slice have been delivered everywhere.
  __syncthreads();
  if (threadIdx.x == 0) {
    fence_sys();
    nvls::red_release_add_u32(reinterpret_cast<void*>(mc_base + counter_off), 1u);
    wait_until_ge(my_counter, target0 + (uint32_t)(gridDim.x * world), timeout_ns,
                  reinterpret_cast<StatusBlock*>(hb[rank] + status_off), 81, (uint32_t)rank, 1);
    all_reduce_leave(my_counter, base, world);
  }
}

}  // namespace

extern "C" {

int iris_k_nvls_all_store(uint64_t mc_ptr, uint64_t bytes, int grid, int block, void* stream) {
  nvls_all_store_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(mc_ptr, bytes / 16);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

int iris_k_nvls_all_reduce_bf16(uint64_t mc_buf, const uint64_t* hb, uint64_t counter_off, uint64_t status_off,
                                uint64_t bytes, int rank, int world, uint64_t timeout_ns, uint64_t mc_base, int grid,
                                int block, void* stream) {
  nvls_all_reduce_bf16_kernel<<<grid, block, 0, (cudaStream_t)stream>>>(mc_buf, hb, counter_off, status_off, bytes / 16,
                                                                        rank, world, timeout_ns, mc_base);
  return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // extern "C"
