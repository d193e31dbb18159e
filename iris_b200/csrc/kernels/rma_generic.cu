// rma_generic.cu — element-wise application of every device RMA primitive, for every supported element
// type x memory semantics x scope.  This is the GPU half of the unit tests that the reference writes as
// seven small Triton kernels (tests/unittests/test_{load,store,get,put,atomic_add,atomic_cas,atomic_xchg}.py)
// and it doubles as the demonstration that iris.cuh compiles for all those combinations.
#include <cuda_runtime.h>

#include "iris/rma_ops.cuh"

using namespace iris;
using namespace iris::ops;

namespace {

template <class T, Sem S, Scope C>
__global__ void rma_kernel(int op, RmaArgs g) {
  const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < g.n) rma_apply<T, S, C>(op, i, g);
}

template <class T, Sem S, Scope C>
int launch(int op, const RmaArgs& g, int block, cudaStream_t st) {
  if ((op == kAtomicAdd || op == kAtomicSub) && !Traits<T>::can_add) return -2;
  if (op == kAtomicSub && sizeof(T) < 4) return -2;
  if (op == kAtomicCas && !Traits<T>::can_cas) return -2;
  if (op == kAtomicXchg && !Traits<T>::can_xchg) return -2;
  if (g.n <= 0) return 0;
  const int grid = (int)((g.n + block - 1) / block);
  rma_kernel<T, S, C><<<grid, block, 0, st>>>(op, g);
  return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <class T, Sem S>
int by_scope(int op, int scope, const RmaArgs& g, int block, cudaStream_t st) {
  switch (scope) {
    case 0: return launch<T, S, Scope::cta>(op, g, block, st);
    case 1: return launch<T, S, Scope::gpu>(op, g, block, st);
    case 2: return launch<T, S, Scope::sys>(op, g, block, st);
  }
  return -3;
}

template <class T>
int by_sem(int op, int sem, int scope, const RmaArgs& g, int block, cudaStream_t st) {
  switch (sem) {
    case 0: return by_scope<T, Sem::relaxed>(op, scope, g, block, st);
    case 1: return by_scope<T, Sem::acquire>(op, scope, g, block, st);
    case 2: return by_scope<T, Sem::release>(op, scope, g, block, st);
    case 3: return by_scope<T, Sem::acq_rel>(op, scope, g, block, st);
  }
  return -3;
}

}  // namespace

extern "C" {

// Same contract as iris_cpu_rma (csrc/cpu/iris_cpu_backend.cpp); `block` threads per CTA, grid covers n.
// Returns 0, -1 unknown dtype, -2 unsupported (op, dtype), -3 bad sem/scope, -4 launch error.
int iris_k_rma(int op, int dtype, int sem, int scope, void* a, void* b, void* c, int64_t n, const uint64_t* heap_bases,
               int cur, int world, int target, double fvalue, int64_t ivalue, int64_t ivalue2, int block,
               void* stream) {
  RmaArgs g{a, b, c, n, heap_bases, fvalue, ivalue, ivalue2, cur, world, target};
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (block < 1 || block > 1024) return -3;
  switch (dtype) {
    case kI8: return by_sem<int8_t>(op, sem, scope, g, block, st);
    case kI16: return by_sem<int16_t>(op, sem, scope, g, block, st);
    case kI32: return by_sem<int32_t>(op, sem, scope, g, block, st);
    case kI64: return by_sem<long long>(op, sem, scope, g, block, st);
    case kF16: return by_sem<__half>(op, sem, scope, g, block, st);
    case kBF16: return by_sem<__nv_bfloat16>(op, sem, scope, g, block, st);
    case kF32: return by_sem<float>(op, sem, scope, g, block, st);
    case kF64: return by_sem<double>(op, sem, scope, g, block, st);
  }
  return -1;
}

}  // extern "C"
