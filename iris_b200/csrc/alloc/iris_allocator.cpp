// Pluggable device allocator with the torch.cuda.memory.CUDAPluggableAllocator ABI.
//
// Role in the reference: csrc/finegrained_alloc/finegrained_allocator.hip:27-56 — a malloc/free pair that
// torch calls for every device allocation, so that the symmetric heap (and everything else) lands in
// memory other GPUs can reach.  On NVIDIA GPUs every cudaMalloc'd byte is already reachable by peers once
// it is exported, so this allocator's job is: allocate on the requested device without disturbing the
// caller's current device, optionally log, and report failure by returning nullptr (the reference
// exits the process instead, finegrained_allocator.hip:11-16).
// Logging is switched on by the environment variable LOG_IRIS_ALLOCATOR (any value).
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <sys/types.h>

namespace {
bool logging_enabled() {
  static const bool on = getenv("LOG_IRIS_ALLOCATOR") != nullptr;
  return on;
}
struct DeviceGuard {
  int prev = -1;
  bool switched = false;
  explicit DeviceGuard(int device) {
    if (cudaGetDevice(&prev) == cudaSuccess && prev != device) switched = cudaSetDevice(device) == cudaSuccess;
  }
  ~DeviceGuard() {
    if (switched) cudaSetDevice(prev);
  }
};
}  // namespace

extern "C" {

void* iris_malloc(ssize_t size, int device, cudaStream_t stream) {
  (void)stream;
  DeviceGuard guard(device);
  void* p = nullptr;
  cudaError_t e = cudaMalloc(&p, (size_t)size);
  if (e != cudaSuccess) {
    fprintf(stderr, "[iris allocator] cudaMalloc(%zd) on device %d failed: %s\n", size, device,
            cudaGetErrorString(e));
    (void)cudaGetLastError();
    return nullptr;
  }
  if (logging_enabled()) fprintf(stderr, "[iris allocator] malloc %zd bytes on device %d -> %p\n", size, device, p);
  return p;
}

void iris_free(void* ptr, ssize_t size, int device, cudaStream_t stream) {
  (void)stream;
  DeviceGuard guard(device);
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) {
    fprintf(stderr, "[iris allocator] cudaFree(%p) on device %d failed: %s\n", ptr, device, cudaGetErrorString(e));
    (void)cudaGetLastError();
  }
  if (logging_enabled()) fprintf(stderr, "[iris allocator] free %zd bytes on device %d at %p\n", size, device, ptr);
}

}  // extern "C"
