// rma_ops.cuh — one generic "apply an RMA primitive element-wise" body, shared by the GPU kernels in
// csrc/kernels/rma_generic.cu and by the CPU shared-memory back end (csrc/cpu/iris_cpu_backend.cpp).
//
// The semantics follow the reference's unit-test kernels (tests/unittests/test_load.py:8-31,
// test_store.py:8-30, test_get.py:12-35, test_put.py:12-29, test_atomic_add.py:8-28,
// test_atomic_cas.py:8-23, test_atomic_xchg.py:8-22): with target < 0 the primitive is applied to EVERY
// rank including the caller; with target >= 0 only to that rank.
#pragma once
#include "iris.cuh"

namespace iris {
namespace ops {

enum Op : int {
  kLoad = 0,        // c[i] = sum over targets of load(a + i)
  kStore = 1,       // store(a + i, value) on every target
  kGet = 2,         // get(a + i -> b + i) from every target; c[i] = sum of what arrived
  kPut = 3,         // put(a + i (local) -> b + i (symmetric)) on every target
  kAtomicAdd = 4,   // old = atomic_add(a + i, value); c[i] = old (when c != null)
  kAtomicSub = 5,
  kAtomicCas = 6,   // old = atomic_cas(a + i, compare, value2)
  kAtomicXchg = 7,  // old = atomic_xchg(a + i, value)
};

enum DType : int { kI8 = 0, kI16 = 1, kI32 = 2, kI64 = 3, kF16 = 4, kBF16 = 5, kF32 = 6, kF64 = 7 };

struct RmaArgs {
  void* a;
  void* b;
  void* c;
  int64_t n;
  const uint64_t* heap_bases;
  double fvalue;    // scalar operand for floating types
  int64_t ivalue;   // scalar operand for integer types; `compare` for CAS
  int64_t ivalue2;  // `value` for CAS
  int cur;
  int world;
  int target;  // < 0: all ranks
};

template <class T>
IRIS_HD T scalar_as(double f, int64_t i) {
  if constexpr (std::is_integral<T>::value) {
    return (T)i;
  } else {
    return (T)f;
  }
}
#if defined(__CUDACC__)
template <>
IRIS_HD __half scalar_as<__half>(double f, int64_t) { return __float2half((float)f); }
template <>
IRIS_HD __nv_bfloat16 scalar_as<__nv_bfloat16>(double f, int64_t) { return __float2bfloat16((float)f); }
#endif

template <class T>
IRIS_HD T add_values(T x, T y) { return (T)(x + y); }
#if defined(__CUDACC__)
template <>
IRIS_HD __half add_values<__half>(__half x, __half y) { return __float2half(__half2float(x) + __half2float(y)); }
template <>
IRIS_HD __nv_bfloat16 add_values<__nv_bfloat16>(__nv_bfloat16 x, __nv_bfloat16 y) {
  return __float2bfloat16(__bfloat162float(x) + __bfloat162float(y));
}
#endif

template <class T>
struct Traits {
  static constexpr bool is_int = std::is_integral<T>::value;
  static constexpr bool can_add = sizeof(T) >= 4;                       // 32/64-bit ints, fp32, fp64
  static constexpr bool can_xchg = sizeof(T) >= 4;
  static constexpr bool can_cas = is_int && sizeof(T) >= 2;
};
#if defined(__CUDACC__)
template <> struct Traits<__half> {
  static constexpr bool is_int = false, can_add = true, can_xchg = false, can_cas = false;
};
template <> struct Traits<__nv_bfloat16> {
  static constexpr bool is_int = false, can_add = true, can_xchg = false, can_cas = false;
};
#endif

// Returns false when the (op, type) pair is not supported.
template <class T, Sem S, Scope C>
IRIS_HD bool rma_apply(int op, int64_t i, const RmaArgs& g) {
  T* a = (T*)g.a;
  T* b = (T*)g.b;
  T* c = (T*)g.c;
  const int t0 = g.target < 0 ? 0 : g.target;
  const int t1 = g.target < 0 ? g.world : g.target + 1;
  const T value = scalar_as<T>(g.fvalue, g.ivalue);
  switch (op) {
    case kLoad: {
      T acc = scalar_as<T>(0.0, 0);
      for (int t = t0; t < t1; ++t) acc = add_values(acc, load(a + i, g.cur, t, g.heap_bases));
      c[i] = acc;
      return true;
    }
    case kStore:
      for (int t = t0; t < t1; ++t) store(a + i, value, g.cur, t, g.heap_bases);
      return true;
    case kGet: {
      T acc = scalar_as<T>(0.0, 0);
      for (int t = t0; t < t1; ++t) {
        get(a + i, b + i, g.cur, t, g.heap_bases);
        acc = add_values(acc, b[i]);
      }
      c[i] = acc;
      return true;
    }
    case kPut:
      for (int t = t0; t < t1; ++t) put(a + i, b + i, g.cur, t, g.heap_bases);
      return true;
    case kAtomicAdd:
    case kAtomicSub:
      if constexpr (Traits<T>::can_add) {
        T old = value;
        for (int t = t0; t < t1; ++t) {
          if (op == kAtomicAdd) old = atomic_add<S, C>(a + i, value, g.cur, t, g.heap_bases);
          else {
            if constexpr (sizeof(T) >= 4) old = atomic_sub<S, C>(a + i, value, g.cur, t, g.heap_bases);
            else return false;
          }
        }
        if (c) c[i] = old;
        return true;
      } else {
        return false;
      }
    case kAtomicCas:
      if constexpr (Traits<T>::can_cas) {
        T old = value;
        for (int t = t0; t < t1; ++t)
          old = atomic_cas<S, C>(a + i, (T)g.ivalue, (T)g.ivalue2, g.cur, t, g.heap_bases);
        if (c) c[i] = old;
        return true;
      } else {
        return false;
      }
    case kAtomicXchg:
      if constexpr (Traits<T>::can_xchg) {
        T old = value;
        for (int t = t0; t < t1; ++t) old = atomic_xchg<S, C>(a + i, value, g.cur, t, g.heap_bases);
        if (c) c[i] = old;
        return true;
      } else {
        return false;
      }
  }
  return false;
}

}  // namespace ops
}  // namespace iris
