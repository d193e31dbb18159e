// iris.cuh — device-side RMA API for a symmetric heap shared by the GPUs of one NVLink/NVSwitch box.
//
// Every rank owns one heap; every rank maps every other rank's heap into its own address space and
// keeps the table of those base addresses (`heap_bases`, uint64[world]) in device memory.  A "symmetric
// pointer" is an ordinary pointer into the caller's own heap; the functions below rebase it into the
// target rank's heap and issue a plain load / store / atomic there, which the fabric carries out.
//
// Parity with the reference device API (iris/iris.py:317-521): translate, load, store, get, put,
// atomic_add, atomic_sub, atomic_cas, atomic_xchg with the same argument order
// (ptr..., cur_rank, target_rank, heap_bases, mask -> pred, sem, scope).  A Triton "block of lanes with a
// mask" becomes "one thread with a predicate".  Extensions (16-byte vector forms, block-cooperative
// copies, flags with bounded waits, a nanosecond timer) serve the fused GEMM+collective kernels.
//
// The same header compiles as plain host C++ (no nvcc): the memory operations then map onto GCC
// __atomic builtins, which is what the CPU shared-memory back end uses for the multi-process tests.
#pragma once
#include <stdint.h>
#include <stddef.h>
#include <type_traits>

#if defined(__CUDACC__)
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#define IRIS_HD __host__ __device__ __forceinline__
#define IRIS_DEV __device__ __forceinline__
#else
#include <string.h>
#define IRIS_HD inline
#define IRIS_DEV inline
#endif

#if defined(__CUDA_ARCH__)
#define IRIS_ON_DEVICE 1
#else
#define IRIS_ON_DEVICE 0
#endif

namespace iris {

// Memory-ordering semantics and visibility scope of an atomic, as in the reference's
// sem ∈ {relaxed, acquire, release, acq_rel} and scope ∈ {cta, gpu, sys} (iris/iris.py:429-521).
enum class Sem : int { relaxed = 0, acquire = 1, release = 2, acq_rel = 3 };
enum class Scope : int { cta = 0, gpu = 1, sys = 2 };

// Status codes written by bounded waits and (in the checking build) by translate.
enum Status : uint32_t { kOk = 0, kTimeout = 1, kBadPointer = 2, kBadRank = 3 };

// A record that the first failing wait / check of a kernel fills in; the host reads it after the launch.
struct StatusBlock {
  uint32_t code;    // Status
  uint32_t where;   // caller-chosen site id
  uint32_t rank;    // rank that recorded it
  uint32_t detail;  // e.g. tile index
  uint64_t value;   // e.g. last flag value seen, or the offending address
  uint64_t aux;
};

// Everything a kernel needs to talk to its peers, passed by value.
struct Context {
  const uint64_t* heap_bases;  // device table: base address, in this process, of every rank's heap
  uint64_t heap_size;          // bytes per rank
  uint64_t mc_base;            // NVLS multicast address of the heap, or 0 when not bound
  StatusBlock* status;         // may be null
  int rank;
  int world;
};

// ------------------------------------------------------------------------------------------------
// translate — reference: iris/iris.py:318-339
// ------------------------------------------------------------------------------------------------
template <class T>
IRIS_HD T* translate(T* ptr, int cur_rank, int target_rank, const uint64_t* heap_bases) {
  const uint64_t off = reinterpret_cast<uint64_t>(ptr) - heap_bases[cur_rank];
  return reinterpret_cast<T*>(heap_bases[target_rank] + off);
}

// Checking variant: verifies that the pointer lies in the caller's heap and that the rank exists.
// A violation is recorded in `st` (first one wins) and the function returns nullptr instead of a
// pointer, so the caller can skip the access; it never traps.
template <class T>
IRIS_HD T* translate_checked(T* ptr, const Context& c, int target_rank, uint32_t where = 0);

#if defined(__CUDACC__)
// ------------------------------------------------------------------------------------------------
// Device: timer
// ------------------------------------------------------------------------------------------------
// Nanosecond wall clock shared by all SMs (the analogue of the reference's s_memrealtime reader,
// examples/common/utils.py:135-147).  Rate: 1 GHz.
IRIS_DEV uint64_t globaltimer() {
  uint64_t t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#endif

IRIS_HD void record_status(StatusBlock* st, uint32_t code, uint32_t where, uint32_t rank, uint32_t detail,
                           uint64_t value, uint64_t aux = 0) {
  if (!st) return;
#if IRIS_ON_DEVICE
  if (atomicCAS(&st->code, 0u, code) == 0u) {
#else
  uint32_t expect = 0;
  if (__atomic_compare_exchange_n(&st->code, &expect, code, false, __ATOMIC_ACQ_REL, __ATOMIC_ACQUIRE)) {
#endif
    st->where = where;
    st->rank = rank;
    st->detail = detail;
    st->value = value;
    st->aux = aux;
  }
}

template <class T>
IRIS_HD T* translate_checked(T* ptr, const Context& c, int target_rank, uint32_t where) {
  const uint64_t p = reinterpret_cast<uint64_t>(ptr);
  const uint64_t base = c.heap_bases[c.rank];
  if (target_rank < 0 || target_rank >= c.world) {
    record_status(c.status, kBadRank, where, (uint32_t)c.rank, (uint32_t)target_rank, p);
    return nullptr;
  }
  if (p < base || p >= base + c.heap_size) {
    record_status(c.status, kBadPointer, where, (uint32_t)c.rank, (uint32_t)target_rank, p, base);
    return nullptr;
  }
  return reinterpret_cast<T*>(c.heap_bases[target_rank] + (p - base));
}

// ------------------------------------------------------------------------------------------------
// Plain accesses: load / store / get / put — reference: iris/iris.py:343-425
// ------------------------------------------------------------------------------------------------
template <class T>
IRIS_HD T load(const T* src_ptr, int cur_rank, int target_rank, const uint64_t* heap_bases, bool pred = true) {
  T v{};
  if (pred) v = *translate(src_ptr, cur_rank, target_rank, heap_bases);
  return v;
}

// Note the reference's naming: the first argument of `store` is the destination.
template <class T>
IRIS_HD void store(T* dst_ptr, T data, int cur_rank, int target_rank, const uint64_t* heap_bases,
                   bool pred = true) {
  if (pred) *translate(dst_ptr, cur_rank, target_rank, heap_bases) = data;
}

// get: remote src -> local dst.
template <class T>
IRIS_HD void get(const T* src_ptr, T* dst_ptr, int cur_rank, int target_rank, const uint64_t* heap_bases,
                 bool pred = true) {
  if (pred) *dst_ptr = *translate(src_ptr, cur_rank, target_rank, heap_bases);
}

// put: local src -> remote dst.
template <class T>
IRIS_HD void put(const T* src_ptr, T* dst_ptr, int cur_rank, int target_rank, const uint64_t* heap_bases,
                 bool pred = true) {
  if (pred) *translate(dst_ptr, cur_rank, target_rank, heap_bases) = *src_ptr;
}

// ------------------------------------------------------------------------------------------------
// Atomics
// ------------------------------------------------------------------------------------------------
namespace detail {

#if !IRIS_ON_DEVICE
template <Sem S>
inline int host_order() {
  return S == Sem::relaxed ? __ATOMIC_RELAXED
       : S == Sem::acquire ? __ATOMIC_ACQUIRE
       : S == Sem::release ? __ATOMIC_RELEASE
                           : __ATOMIC_ACQ_REL;
}
#endif

template <int N> struct BitsOf;
template <> struct BitsOf<2> { using type = uint16_t; };
template <> struct BitsOf<4> { using type = uint32_t; };
template <> struct BitsOf<8> { using type = uint64_t; };

template <class To, class From>
IRIS_HD To bit_cast(const From& f) {
  static_assert(sizeof(To) == sizeof(From), "bit_cast size mismatch");
  To t;
#if IRIS_ON_DEVICE
  t = *reinterpret_cast<const To*>(&f);
#else
  memcpy(&t, &f, sizeof(To));
#endif
  return t;
}

#if defined(__CUDACC__)
// One `atom` instruction per (semantics, scope); the macro argument is the tail of the instruction
// starting at ".global".  Expands to a constexpr-if chain so that exactly one asm statement survives.
#define IRIS_ATOM_ONE(SEM, SCOPE, SEMSTR, SCOPESTR, TAIL, OUTC, INC, ...)                              \
  if constexpr (S == Sem::SEM && C == Scope::SCOPE) {                                                  \
    asm volatile("atom." SEMSTR "." SCOPESTR TAIL : OUTC(old) : "l"(p), __VA_ARGS__ : "memory");       \
  }
#define IRIS_ATOM_ALL(TAIL, OUTC, INC, ...)                                                            \
  IRIS_ATOM_ONE(relaxed, cta, "relaxed", "cta", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(relaxed, gpu, "relaxed", "gpu", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(relaxed, sys, "relaxed", "sys", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acquire, cta, "acquire", "cta", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acquire, gpu, "acquire", "gpu", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acquire, sys, "acquire", "sys", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(release, cta, "release", "cta", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(release, gpu, "release", "gpu", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(release, sys, "release", "sys", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acq_rel, cta, "acq_rel", "cta", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acq_rel, gpu, "acq_rel", "gpu", TAIL, OUTC, INC, __VA_ARGS__)                          \
  IRIS_ATOM_ONE(acq_rel, sys, "acq_rel", "sys", TAIL, OUTC, INC, __VA_ARGS__)

template <Sem S, Scope C>
__device__ __forceinline__ uint32_t atom_add_u32(uint32_t* p, uint32_t v) {
  uint32_t old = 0;
  IRIS_ATOM_ALL(".global.add.u32 %0, [%1], %2;", "=r", "r", "r"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint64_t atom_add_u64(uint64_t* p, uint64_t v) {
  uint64_t old = 0;
  IRIS_ATOM_ALL(".global.add.u64 %0, [%1], %2;", "=l", "l", "l"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ float atom_add_f32(float* p, float v) {
  float old = 0.f;
  IRIS_ATOM_ALL(".global.add.f32 %0, [%1], %2;", "=f", "f", "f"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ double atom_add_f64(double* p, double v) {
  double old = 0.;
  IRIS_ATOM_ALL(".global.add.f64 %0, [%1], %2;", "=d", "d", "d"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint16_t atom_add_f16(uint16_t* p, uint16_t v) {
  uint16_t old = 0;
  IRIS_ATOM_ALL(".global.add.noftz.f16 %0, [%1], %2;", "=h", "h", "h"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint16_t atom_add_bf16(uint16_t* p, uint16_t v) {
  uint16_t old = 0;
  IRIS_ATOM_ALL(".global.add.noftz.bf16 %0, [%1], %2;", "=h", "h", "h"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint32_t atom_exch_b32(uint32_t* p, uint32_t v) {
  uint32_t old = 0;
  IRIS_ATOM_ALL(".global.exch.b32 %0, [%1], %2;", "=r", "r", "r"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint64_t atom_exch_b64(uint64_t* p, uint64_t v) {
  uint64_t old = 0;
  IRIS_ATOM_ALL(".global.exch.b64 %0, [%1], %2;", "=l", "l", "l"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint16_t atom_cas_b16(uint16_t* p, uint16_t cmp, uint16_t v) {
  uint16_t old = 0;
  IRIS_ATOM_ALL(".global.cas.b16 %0, [%1], %2, %3;", "=h", "h", "h"(cmp), "h"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint32_t atom_cas_b32(uint32_t* p, uint32_t cmp, uint32_t v) {
  uint32_t old = 0;
  IRIS_ATOM_ALL(".global.cas.b32 %0, [%1], %2, %3;", "=r", "r", "r"(cmp), "r"(v))
  return old;
}
template <Sem S, Scope C>
__device__ __forceinline__ uint64_t atom_cas_b64(uint64_t* p, uint64_t cmp, uint64_t v) {
  uint64_t old = 0;
  IRIS_ATOM_ALL(".global.cas.b64 %0, [%1], %2, %3;", "=l", "l", "l"(cmp), "l"(v))
  return old;
}
#undef IRIS_ATOM_ALL
#undef IRIS_ATOM_ONE
#endif  // __CUDACC__

// ---- dispatch on element type ----
template <Sem S, Scope C, class T>
IRIS_HD T fetch_add(T* p, T v) {
#if IRIS_ON_DEVICE
  if constexpr (sizeof(T) == 4 && std::is_integral<T>::value) {
    return (T)atom_add_u32<S, C>((uint32_t*)p, (uint32_t)v);
  } else if constexpr (sizeof(T) == 8 && std::is_integral<T>::value) {
    return (T)atom_add_u64<S, C>((uint64_t*)p, (uint64_t)v);
  } else if constexpr (sizeof(T) == 4) {
    return atom_add_f32<S, C>((float*)p, (float)v);
  } else {
    static_assert(sizeof(T) == 8, "unsupported type for atomic add");
    return atom_add_f64<S, C>((double*)p, (double)v);
  }
#else
  if constexpr (std::is_integral<T>::value) {
    return __atomic_fetch_add(p, v, host_order<S>());
  } else {
    using B = typename BitsOf<sizeof(T)>::type;
    B* bp = reinterpret_cast<B*>(p);
    B cur = __atomic_load_n(bp, __ATOMIC_RELAXED);
    for (;;) {
      T nv = bit_cast<T>(cur) + v;
      if (__atomic_compare_exchange_n(bp, &cur, bit_cast<B>(nv), true, host_order<S>(), __ATOMIC_RELAXED))
        return bit_cast<T>(cur);
    }
  }
#endif
}

#if defined(__CUDACC__)
template <Sem S, Scope C>
IRIS_HD __half fetch_add(__half* p, __half v) {
#if IRIS_ON_DEVICE
  return bit_cast<__half>(atom_add_f16<S, C>((uint16_t*)p, bit_cast<uint16_t>(v)));
#else
  uint16_t* bp = reinterpret_cast<uint16_t*>(p);
  uint16_t cur = __atomic_load_n(bp, __ATOMIC_RELAXED);
  for (;;) {
    __half nv = __float2half(__half2float(bit_cast<__half>(cur)) + __half2float(v));
    if (__atomic_compare_exchange_n(bp, &cur, bit_cast<uint16_t>(nv), true, host_order<S>(), __ATOMIC_RELAXED))
      return bit_cast<__half>(cur);
  }
#endif
}
template <Sem S, Scope C>
IRIS_HD __nv_bfloat16 fetch_add(__nv_bfloat16* p, __nv_bfloat16 v) {
#if IRIS_ON_DEVICE
  return bit_cast<__nv_bfloat16>(atom_add_bf16<S, C>((uint16_t*)p, bit_cast<uint16_t>(v)));
#else
  uint16_t* bp = reinterpret_cast<uint16_t*>(p);
  uint16_t cur = __atomic_load_n(bp, __ATOMIC_RELAXED);
  for (;;) {
    __nv_bfloat16 nv = __float2bfloat16(__bfloat162float(bit_cast<__nv_bfloat16>(cur)) + __bfloat162float(v));
    if (__atomic_compare_exchange_n(bp, &cur, bit_cast<uint16_t>(nv), true, host_order<S>(), __ATOMIC_RELAXED))
      return bit_cast<__nv_bfloat16>(cur);
  }
#endif
}
#endif

template <Sem S, Scope C, class T>
IRIS_HD T exchange(T* p, T v) {
  using B = typename BitsOf<sizeof(T)>::type;
#if IRIS_ON_DEVICE
  if constexpr (sizeof(T) == 4) {
    return bit_cast<T>(atom_exch_b32<S, C>((uint32_t*)p, bit_cast<uint32_t>(v)));
  } else {
    static_assert(sizeof(T) == 8, "atomic_xchg supports 32- and 64-bit types");
    return bit_cast<T>(atom_exch_b64<S, C>((uint64_t*)p, bit_cast<uint64_t>(v)));
  }
#else
  return bit_cast<T>(__atomic_exchange_n(reinterpret_cast<B*>(p), bit_cast<B>(v), host_order<S>()));
#endif
}

template <Sem S, Scope C, class T>
IRIS_HD T compare_swap(T* p, T cmp, T v) {
  using B = typename BitsOf<sizeof(T)>::type;
#if IRIS_ON_DEVICE
  if constexpr (sizeof(T) == 2) {
    return bit_cast<T>(atom_cas_b16<S, C>((uint16_t*)p, bit_cast<uint16_t>(cmp), bit_cast<uint16_t>(v)));
  } else if constexpr (sizeof(T) == 4) {
    return bit_cast<T>(atom_cas_b32<S, C>((uint32_t*)p, bit_cast<uint32_t>(cmp), bit_cast<uint32_t>(v)));
  } else {
    static_assert(sizeof(T) == 8, "atomic_cas supports 16-, 32- and 64-bit types");
    return bit_cast<T>(atom_cas_b64<S, C>((uint64_t*)p, bit_cast<uint64_t>(cmp), bit_cast<uint64_t>(v)));
  }
#else
  B expect = bit_cast<B>(cmp);
  // A failed CAS only needs the load half of the ordering.
  const int fail = (S == Sem::relaxed || S == Sem::release) ? __ATOMIC_RELAXED : __ATOMIC_ACQUIRE;
  __atomic_compare_exchange_n(reinterpret_cast<B*>(p), &expect, bit_cast<B>(v), false, host_order<S>(), fail);
  return bit_cast<T>(expect);
#endif
}

}  // namespace detail

// atomic_add / atomic_sub / atomic_xchg / atomic_cas — reference: iris/iris.py:429-521.
// Defaults match the reference (sem = acq_rel, scope = gpu).  All return the previous value.
template <Sem S = Sem::acq_rel, Scope C = Scope::gpu, class T>
IRIS_HD T atomic_add(T* ptr, T data, int cur_rank, int target_rank, const uint64_t* heap_bases, bool pred = true) {
  if (!pred) return T{};
  return detail::fetch_add<S, C>(translate(ptr, cur_rank, target_rank, heap_bases), data);
}
template <Sem S = Sem::acq_rel, Scope C = Scope::gpu, class T>
IRIS_HD T atomic_sub(T* ptr, T data, int cur_rank, int target_rank, const uint64_t* heap_bases, bool pred = true) {
  if (!pred) return T{};
  return detail::fetch_add<S, C>(translate(ptr, cur_rank, target_rank, heap_bases), (T)(-data));
}
template <Sem S = Sem::acq_rel, Scope C = Scope::gpu, class T>
IRIS_HD T atomic_xchg(T* ptr, T value, int cur_rank, int target_rank, const uint64_t* heap_bases, bool pred = true) {
  if (!pred) return T{};
  return detail::exchange<S, C>(translate(ptr, cur_rank, target_rank, heap_bases), value);
}
template <Sem S = Sem::acq_rel, Scope C = Scope::gpu, class T>
IRIS_HD T atomic_cas(T* ptr, T compare, T value, int cur_rank, int target_rank, const uint64_t* heap_bases) {
  return detail::compare_swap<S, C>(translate(ptr, cur_rank, target_rank, heap_bases), compare, value);
}

// ------------------------------------------------------------------------------------------------
// Flags: release/acquire signalling with bounded waits (extension; the reference spins without bound,
// examples/09_gemm_one_shot_all_reduce/gemm_one_shot_all_reduce.py:220-234).
// ------------------------------------------------------------------------------------------------
IRIS_HD uint32_t ld_acquire_sys(const uint32_t* p) {
#if IRIS_ON_DEVICE
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n(p, __ATOMIC_ACQUIRE);
#endif
}
IRIS_HD uint32_t ld_relaxed_sys(const uint32_t* p) {
#if IRIS_ON_DEVICE
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
#else
  return __atomic_load_n(p, __ATOMIC_RELAXED);
#endif
}
IRIS_HD void st_release_sys(uint32_t* p, uint32_t v) {
#if IRIS_ON_DEVICE
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
  __atomic_store_n(p, v, __ATOMIC_RELEASE);
#endif
}
IRIS_HD void st_relaxed_sys(uint32_t* p, uint32_t v) {
#if IRIS_ON_DEVICE
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
  __atomic_store_n(p, v, __ATOMIC_RELAXED);
#endif
}
IRIS_HD void red_release_sys_add(uint32_t* p, uint32_t v) {
#if IRIS_ON_DEVICE
  asm volatile("red.release.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
  __atomic_fetch_add(p, v, __ATOMIC_RELEASE);
#endif
}
IRIS_HD void red_relaxed_sys_add(uint32_t* p, uint32_t v) {
#if IRIS_ON_DEVICE
  asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
#else
  __atomic_fetch_add(p, v, __ATOMIC_RELAXED);
#endif
}
IRIS_HD void fence_sys() {
#if IRIS_ON_DEVICE
  asm volatile("fence.acq_rel.sys;" ::: "memory");
#else
  __atomic_thread_fence(__ATOMIC_SEQ_CST);
#endif
}

// signal: add `v` to the flag at the same offset in `target_rank`'s heap, releasing all earlier writes
// of this thread (and, through a preceding barrier, of its block) at system scope.
IRIS_HD void signal_add(uint32_t* flag, uint32_t v, int cur_rank, int target_rank, const uint64_t* heap_bases) {
  red_release_sys_add(translate(flag, cur_rank, target_rank, heap_bases), v);
}
// signal_set: store `v` into the remote flag with release semantics.
IRIS_HD void signal_set(uint32_t* flag, uint32_t v, int cur_rank, int target_rank, const uint64_t* heap_bases) {
  st_release_sys(translate(flag, cur_rank, target_rank, heap_bases), v);
}

// wait_until_ge: poll a LOCAL flag with acquire loads until it reaches `expected` (wrap-safe signed
// comparison) or `timeout_ns` elapses.  On expiry it records {kTimeout, where, rank, detail, last value}
// in `st` and returns kTimeout; it never traps and never spins without bound.
IRIS_HD uint32_t wait_until_ge(const uint32_t* flag, uint32_t expected, uint64_t timeout_ns,
                               StatusBlock* st = nullptr, uint32_t where = 0, uint32_t rank = 0,
                               uint32_t detail = 0) {
  uint32_t v = ld_acquire_sys(flag);
  if ((int32_t)(v - expected) >= 0) return kOk;
#if IRIS_ON_DEVICE
  const uint64_t t0 = globaltimer();
  uint32_t backoff = 32;
  for (;;) {
    v = ld_acquire_sys(flag);
    if ((int32_t)(v - expected) >= 0) return kOk;
    if (globaltimer() - t0 > timeout_ns) break;
    __nanosleep(backoff);
    if (backoff < 1024) backoff <<= 1;
  }
#else
  // Host: a bounded number of polls; one poll is of the order of a nanosecond to a microsecond.
  for (uint64_t i = 0; i < timeout_ns; ++i) {
    v = ld_acquire_sys(flag);
    if ((int32_t)(v - expected) >= 0) return kOk;
    if ((i & 1023) == 1023) {
      __builtin_ia32_pause();
    }
  }
#endif
  record_status(st, kTimeout, where, rank, detail, v, expected);
  return kTimeout;
}

#if defined(__CUDACC__)
// ------------------------------------------------------------------------------------------------
// 16-byte vector forms and block-cooperative copies (extensions used by the bandwidth kernels).
// ------------------------------------------------------------------------------------------------
IRIS_DEV uint4 ld_v4(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
  return v;
}
// Streaming load that does not allocate in L1 (remote data is read once).
IRIS_DEV uint4 ld_v4_stream(const uint4* p) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p));
  return v;
}
IRIS_DEV void st_v4(uint4* p, uint4 v) {
  asm volatile("st.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w) : "memory");
}

IRIS_DEV uint4 load_v4(const uint4* src, int cur, int tgt, const uint64_t* hb) {
  return ld_v4_stream(translate(src, cur, tgt, hb));
}
IRIS_DEV void store_v4(uint4* dst, uint4 v, int cur, int tgt, const uint64_t* hb) {
  st_v4(translate(dst, cur, tgt, hb), v);
}

// Whole-block copy of `bytes` (multiple of 16, both pointers 16-byte aligned) from the caller's heap to
// the same offset range in `target_rank`'s heap (put) or the reverse (get).  Four 16-byte accesses are
// kept in flight per thread.
IRIS_DEV void copy_block_16B(uint4* dst, const uint4* src, size_t n16) {
  const size_t stride = blockDim.x;
  size_t i = threadIdx.x;
  for (; i + 3 * stride < n16; i += 4 * stride) {
    uint4 a = ld_v4_stream(src + i);
    uint4 b = ld_v4_stream(src + i + stride);
    uint4 c = ld_v4_stream(src + i + 2 * stride);
    uint4 d = ld_v4_stream(src + i + 3 * stride);
    st_v4(dst + i, a);
    st_v4(dst + i + stride, b);
    st_v4(dst + i + 2 * stride, c);
    st_v4(dst + i + 3 * stride, d);
  }
  for (; i < n16; i += stride) st_v4(dst + i, ld_v4_stream(src + i));
}
IRIS_DEV void put_block(const void* local_src, void* sym_dst, size_t bytes, int cur, int tgt, const uint64_t* hb) {
  copy_block_16B(translate((uint4*)sym_dst, cur, tgt, hb), (const uint4*)local_src, bytes / 16);
}
IRIS_DEV void get_block(const void* sym_src, void* local_dst, size_t bytes, int cur, int tgt, const uint64_t* hb) {
  copy_block_16B((uint4*)local_dst, translate((const uint4*)sym_src, cur, tgt, hb), bytes / 16);
}

// Non-returning vector reductions into global memory (any mapped address, peers included).
IRIS_DEV void red_add_v4_f32(float* p, float a, float b, float c, float d) {
  asm volatile("red.relaxed.sys.global.add.v4.f32 [%0], {%1,%2,%3,%4};" ::"l"(p), "f"(a), "f"(b), "f"(c), "f"(d)
               : "memory");
}
IRIS_DEV void red_add_v4_bf16x2(void* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("red.relaxed.sys.global.add.noftz.v4.bf16x2 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(a), "r"(b), "r"(c),
               "r"(d)
               : "memory");
}
IRIS_DEV void red_add_f32(float* p, float a) {
  asm volatile("red.relaxed.sys.global.add.f32 [%0], %1;" ::"l"(p), "f"(a) : "memory");
}
#endif  // __CUDACC__

}  // namespace iris
