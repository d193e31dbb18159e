// nvls.cuh — NVLink-switch multicast ("NVLS") instructions on a heap bound to a multicast object.
//
// An address inside the multicast mapping of the heap (Context::mc_base + offset) names the same offset in
// EVERY rank's heap at once:
//   multimem.st         one store, delivered by the switch to all ranks (egress 1x instead of (W-1)x);
//   multimem.red        one reduction, applied to every rank's copy;
//   multimem.ld_reduce  one load that returns the sum over all ranks' copies, added inside the switch.
// The reference has nothing of the kind (its fabric has no switch); these are the B200 answer to its
// all-store / atomic all-reduce patterns (examples/03_all_store, examples/08_gemm_atomics_all_reduce).
// The libcu++ wrappers cover only integer forms, so the floating-point forms are spelled out here.
#pragma once
#include <stdint.h>

#include "iris.cuh"

namespace iris {
namespace nvls {

// Translate a symmetric pointer into the multicast mapping.
template <class T>
__device__ __forceinline__ T* multicast_ptr(T* sym_ptr, const Context& c) {
  return reinterpret_cast<T*>(c.mc_base + (reinterpret_cast<uint64_t>(sym_ptr) - c.heap_bases[c.rank]));
}

__device__ __forceinline__ void st_v4(void* mc, uint4 v) {
  asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y), "r"(v.z),
               "r"(v.w)
               : "memory");
}
__device__ __forceinline__ void st_u32(void* mc, uint32_t v) {
  asm volatile("multimem.st.relaxed.sys.global.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
// Release-add on the same flag word of every rank.
__device__ __forceinline__ void red_release_add_u32(void* mc, uint32_t v) {
  asm volatile("multimem.red.release.sys.global.add.u32 [%0], %1;" ::"l"(mc), "r"(v) : "memory");
}
// 8 bf16 summed over all ranks with fp32 accumulation inside the switch.
__device__ __forceinline__ uint4 ld_reduce_add_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// The same for 8 fp16 values.
__device__ __forceinline__ uint4 ld_reduce_add_f16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.f16x2 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_reduce_add_f32x4(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}
// Add 8 bf16 into every rank's copy.
__device__ __forceinline__ void red_add_bf16x8(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

// The same for 8 fp16 values.
__device__ __forceinline__ void red_add_f16x8(void* mc, uint4 v) {
  asm volatile("multimem.red.relaxed.sys.global.add.v4.f16x2 [%0], {%1,%2,%3,%4};" ::"l"(mc), "r"(v.x), "r"(v.y),
               "r"(v.z), "r"(v.w)
               : "memory");
}

}  // namespace nvls
}  // namespace iris
