// CPU back end of the symmetric heap: one POSIX shared-memory segment per rank, mapped by every rank,
// and the same RMA primitives as the GPU header (include/iris/iris.cuh compiled as host C++).
//
// Purpose: the host-side plumbing (bootstrap, allocation sequence, base-address table, pointer
// translation, flag protocols, time-outs) can be exercised by several processes on a machine without a
// GPU.  The reference has no such path (it needs HIP at import: iris/_hip.py:8-9); its role here is the
// one that `mpirun -np N pytest` plays for the reference's unit tests (tests/unittests/*.py).
#include <errno.h>
#include <fcntl.h>
#include <stdio.h>
#include <string.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <thread>
#include <vector>

#include "iris/rma_ops.cuh"

using namespace iris;
using namespace iris::ops;

namespace {
thread_local char g_err[256] = "";
void set_err(const char* what) { snprintf(g_err, sizeof(g_err), "%s: %s", what, strerror(errno)); }
}  // namespace

extern "C" {

const char* iris_cpu_last_error() { return g_err; }

// Create (owner) or attach to (peer) the segment `name` of `size` bytes.  Returns the mapping or null.
void* iris_cpu_heap_map(const char* name, uint64_t size, int create) {
  int fd = shm_open(name, create ? (O_CREAT | O_EXCL | O_RDWR) : O_RDWR, 0600);
  if (fd < 0) {
    set_err("shm_open");
    return nullptr;
  }
  if (create && ftruncate(fd, (off_t)size) != 0) {
    set_err("ftruncate");
    close(fd);
    shm_unlink(name);
    return nullptr;
  }
  if (!create) {
    struct stat st;
    if (fstat(fd, &st) != 0 || (uint64_t)st.st_size < size) {
      snprintf(g_err, sizeof(g_err), "segment %s is smaller than %llu bytes", name, (unsigned long long)size);
      close(fd);
      return nullptr;
    }
  }
  void* p = mmap(nullptr, size, PROT_READ | PROT_WRITE, MAP_SHARED, fd, 0);
  close(fd);
  if (p == MAP_FAILED) {
    set_err("mmap");
    if (create) shm_unlink(name);
    return nullptr;
  }
  return p;
}

int iris_cpu_heap_unmap(void* p, uint64_t size) { return munmap(p, size); }
int iris_cpu_heap_unlink(const char* name) { return shm_unlink(name); }

}  // extern "C"

namespace {

template <class T, Sem S>
int run_typed(int op, const RmaArgs& g, int nthreads) {
  // Probe support with element 0 semantics: unsupported pairs are reported before touching memory.
  if ((op == kAtomicAdd || op == kAtomicSub) && !Traits<T>::can_add) return -2;
  if (op == kAtomicCas && !Traits<T>::can_cas) return -2;
  if (op == kAtomicXchg && !Traits<T>::can_xchg) return -2;
  if (nthreads < 1) nthreads = 1;
  if (nthreads == 1 || g.n < nthreads) {
    for (int64_t i = 0; i < g.n; ++i) rma_apply<T, S, Scope::sys>(op, i, g);
    return 0;
  }
  // "Threads of a block": a strided split so that neighbouring elements are handled concurrently.
  std::vector<std::thread> pool;
  for (int t = 0; t < nthreads; ++t)
    pool.emplace_back([=]() {
      for (int64_t i = t; i < g.n; i += nthreads) rma_apply<T, S, Scope::sys>(op, i, g);
    });
  for (auto& th : pool) th.join();
  return 0;
}

template <class T>
int run_sem(int op, int sem, const RmaArgs& g, int nthreads) {
  switch (sem) {
    case 0: return run_typed<T, Sem::relaxed>(op, g, nthreads);
    case 1: return run_typed<T, Sem::acquire>(op, g, nthreads);
    case 2: return run_typed<T, Sem::release>(op, g, nthreads);
    case 3: return run_typed<T, Sem::acq_rel>(op, g, nthreads);
  }
  return -3;
}

}  // namespace

extern "C" {

// Apply primitive `op` (iris::ops::Op) to n elements of type `dtype` (iris::ops::DType).
// Returns 0, -1 for an unknown dtype, -2 for an unsupported (op, dtype) pair, -3 for a bad `sem`.
// `scope` is accepted for signature parity; on the host every atomic is system-wide.
int iris_cpu_rma(int op, int dtype, int sem, int scope, void* a, void* b, void* c, int64_t n,
                 const uint64_t* heap_bases, int cur, int world, int target, double fvalue, int64_t ivalue,
                 int64_t ivalue2, int nthreads) {
  (void)scope;
  RmaArgs g{a, b, c, n, heap_bases, fvalue, ivalue, ivalue2, cur, world, target};
  switch (dtype) {
    case kI8: return run_sem<int8_t>(op, sem, g, nthreads);
    case kI16: return run_sem<int16_t>(op, sem, g, nthreads);
    case kI32: return run_sem<int32_t>(op, sem, g, nthreads);
    case kI64: return run_sem<int64_t>(op, sem, g, nthreads);
    case kF32: return run_sem<float>(op, sem, g, nthreads);
    case kF64: return run_sem<double>(op, sem, g, nthreads);
    // 16-bit floating types move as raw 16-bit words (no arithmetic on the host).
    case kF16:
    case kBF16:
      if (op == kStore || op == kPut) return run_sem<int16_t>(op, sem, g, nthreads);
      return -2;
  }
  return -1;
}

// Checking pointer translation (iris::translate_checked): returns the translated address, or 0 after recording
// kBadPointer / kBadRank in `st` when `ptr` is outside the caller's heap or `target` is not a rank.
uint64_t iris_cpu_translate_checked(uint64_t ptr, const uint64_t* heap_bases, uint64_t heap_size, int rank, int world,
                                    int target, StatusBlock* st) {
  Context c{heap_bases, heap_size, 0, st, rank, world};
  return reinterpret_cast<uint64_t>(translate_checked(reinterpret_cast<char*>(ptr), c, target, /*where=*/90));
}

// Producer side of the message-passing protocol (examples/06): copy `bytes` from local `src` into the
// consumer's `dst`, then raise the consumer's flag to `epoch` with release semantics.
void iris_cpu_mp_produce(const void* src, void* dst_sym, uint64_t bytes, uint32_t* flag_sym, uint32_t epoch,
                         const uint64_t* heap_bases, int cur, int target) {
  memcpy(translate((char*)dst_sym, cur, target, heap_bases), src, bytes);
  signal_set(flag_sym, epoch, cur, target, heap_bases);
}

// Consumer side: bounded wait on the local flag; returns iris::Status.
uint32_t iris_cpu_wait_flag(const uint32_t* flag, uint32_t expected, uint64_t max_polls, StatusBlock* st,
                            uint32_t rank) {
  return wait_until_ge(flag, expected, max_polls, st, /*where=*/1, rank, 0);
}

}  // extern "C"
