// Stress program for the CPU back end of the symmetric heap, meant to be built with -fsanitize=thread and with
// -fsanitize=address,undefined (tests/test_sanitizers_cpu.py builds and runs both).  Two "ranks" are two shared-memory
// segments mapped into this process; threads play the ranks.  Every section ends with a check of values, so the
// program is also a plain functional test.  Exit code 0 = all checks passed.
//
// What it covers: element-wise RMA primitives run by several threads (the "threads of a block" of the back end), the
// message-passing protocol (data written with ordinary stores, flag raised with release, consumer polls with
// acquire, then reads the data: a missing ordering shows up as a data race under the thread sanitizer), concurrent
// atomic adds from both ranks, a bounded wait that expires, the checking pointer translation, and a model of the
// fused GEMM's inbox protocol (cumulative flags, buffers alternating by call parity) run with random delays, the
// all-gather prologue, and the stream-K fix-up with the call counter kept in "device" memory.
#include <stdint.h>
#include <stdio.h>
#include <string.h>
#include <unistd.h>

#include <atomic>
#include <chrono>
#include <thread>
#include <vector>

#include "iris/rma_ops.cuh"
#include "kernels/gemm_schedule.h"

extern "C" {
const char* iris_cpu_last_error();
void* iris_cpu_heap_map(const char* name, uint64_t size, int create);
int iris_cpu_heap_unmap(void* p, uint64_t size);
int iris_cpu_heap_unlink(const char* name);
int iris_cpu_rma(int op, int dtype, int sem, int scope, void* a, void* b, void* c, int64_t n, const uint64_t* heap_bases,
                 int cur, int world, int target, double fvalue, int64_t ivalue, int64_t ivalue2, int nthreads);
uint64_t iris_cpu_translate_checked(uint64_t ptr, const uint64_t* heap_bases, uint64_t heap_size, int rank, int world,
                                    int target, iris::StatusBlock* st);
void iris_cpu_mp_produce(const void* src, void* dst_sym, uint64_t bytes, uint32_t* flag_sym, uint32_t epoch,
                         const uint64_t* heap_bases, int cur, int target);
uint32_t iris_cpu_wait_flag(const uint32_t* flag, uint32_t expected, uint64_t max_polls, iris::StatusBlock* st,
                            uint32_t rank);
}

using namespace iris;
using namespace iris::ops;

static int g_fail = 0;
#define CHECK(cond, ...)                   \
  do {                                     \
    if (!(cond)) {                         \
      fprintf(stderr, "FAILED %s:%d: ", __FILE__, __LINE__); \
      fprintf(stderr, __VA_ARGS__);        \
      fprintf(stderr, "\n");               \
      ++g_fail;                            \
    }                                      \
  } while (0)

int main() {
  constexpr uint64_t kHeap = 1 << 20;
  constexpr int kWorld = 2;
  char name[kWorld][64];
  uint8_t* base[kWorld];
  for (int r = 0; r < kWorld; ++r) {
    snprintf(name[r], sizeof(name[r]), "/iris_stress_%d_%d", (int)getpid(), r);
    base[r] = static_cast<uint8_t*>(iris_cpu_heap_map(name[r], kHeap, 1));
    if (!base[r]) {
      fprintf(stderr, "map: %s\n", iris_cpu_last_error());
      return 2;
    }
    memset(base[r], 0, kHeap);
  }
  const uint64_t hb[kWorld] = {(uint64_t)base[0], (uint64_t)base[1]};
  // The same offsets on every rank: [0, 64K) data A, [64K, 128K) data B, [128K, 192K) results, [192K, ...) flags.
  auto sym = [&](int rank, uint64_t off) { return base[rank] + off; };
  constexpr uint64_t kA = 0, kB = 64 << 10, kC = 128 << 10, kF = 192 << 10;
  constexpr int64_t kN = 4096;

  // ---- 1. element-wise primitives, four threads per call, every memory order ----
  for (int sem = 0; sem < 4; ++sem) {
    // rank 0 stores 7 into A of every rank
    int rc = iris_cpu_rma(kStore, kI32, sem, 2, sym(0, kA), nullptr, nullptr, kN, hb, 0, kWorld, -1, 0.0, 7, 0, 4);
    CHECK(rc == 0, "store rc %d", rc);
    for (int r = 0; r < kWorld; ++r)
      for (int64_t i = 0; i < kN; ++i) CHECK(reinterpret_cast<int32_t*>(sym(r, kA))[i] == 7, "store value");
    // rank 1 loads A from every rank and sums into its C: 7 * world
    rc = iris_cpu_rma(kLoad, kI32, sem, 2, sym(1, kA), nullptr, sym(1, kC), kN, hb, 1, kWorld, -1, 0.0, 0, 0, 4);
    CHECK(rc == 0, "load rc %d", rc);
    CHECK(reinterpret_cast<int32_t*>(sym(1, kC))[kN - 1] == 7 * kWorld, "load sum");
    // rank 0 puts its A into B of rank 1
    rc = iris_cpu_rma(kPut, kI32, sem, 2, sym(0, kA), sym(0, kB), nullptr, kN, hb, 0, kWorld, 1, 0.0, 0, 0, 4);
    CHECK(rc == 0, "put rc %d", rc);
    CHECK(reinterpret_cast<int32_t*>(sym(1, kB))[17] == 7, "put value");
    // fp32 atomic add of 1.5 to C of rank 0 by rank 1, result of the old values ignored
    memset(sym(0, kC), 0, kN * 4);
    rc = iris_cpu_rma(kAtomicAdd, kF32, sem, 2, sym(1, kC), nullptr, nullptr, kN, hb, 1, kWorld, 0, 1.5, 0, 0, 4);
    CHECK(rc == 0, "atomic add rc %d", rc);
    CHECK(reinterpret_cast<float*>(sym(0, kC))[5] == 1.5f, "atomic add value");
    // compare-and-swap 0 -> 9 on int64 words of rank 1
    memset(sym(1, kC), 0, kN * 8);
    rc = iris_cpu_rma(kAtomicCas, kI64, sem, 2, sym(0, kC), nullptr, nullptr, kN, hb, 0, kWorld, 1, 0.0, 0, 9, 4);
    CHECK(rc == 0, "cas rc %d", rc);
    CHECK(reinterpret_cast<int64_t*>(sym(1, kC))[kN - 1] == 9, "cas value");
  }
  CHECK(iris_cpu_rma(kAtomicAdd, kI16, 0, 2, sym(0, kA), nullptr, nullptr, 4, hb, 0, kWorld, 0, 0.0, 1, 0, 1) == -2,
        "16-bit atomic add must be refused");
  CHECK(iris_cpu_rma(kLoad, 99, 0, 2, sym(0, kA), nullptr, nullptr, 4, hb, 0, kWorld, 0, 0.0, 1, 0, 1) == -1,
        "unknown dtype must be refused");

  // ---- 2. both ranks add into the same counters at once ----
  {
    memset(sym(0, kC), 0, kN * 4);
    memset(sym(1, kC), 0, kN * 4);
    std::vector<std::thread> ranks;
    for (int r = 0; r < kWorld; ++r)
      ranks.emplace_back([&, r]() {
        for (int rep = 0; rep < 8; ++rep)
          iris_cpu_rma(kAtomicAdd, kI32, 0, 2, sym(r, kC), nullptr, nullptr, kN, hb, r, kWorld, -1, 0.0, 1, 0, 2);
      });
    for (auto& t : ranks) t.join();
    for (int r = 0; r < kWorld; ++r)
      CHECK(reinterpret_cast<int32_t*>(sym(r, kC))[123] == 8 * kWorld, "concurrent adds: %d",
            reinterpret_cast<int32_t*>(sym(r, kC))[123]);
  }

  // ---- 3. message passing: rank 0 produces 16 chunks for rank 1, which doubles them and sends them back ----
  {
    constexpr int kChunks = 16;
    constexpr uint64_t kChunk = 2048;  // bytes
    std::vector<int32_t> src(kChunks * kChunk / 4), back(kChunks * kChunk / 4);
    for (size_t i = 0; i < src.size(); ++i) src[i] = (int32_t)i;
    uint32_t* flags0 = reinterpret_cast<uint32_t*>(sym(0, kF));
    uint32_t* flags1 = reinterpret_cast<uint32_t*>(sym(1, kF));
    memset(flags0, 0, kChunks * 4);
    memset(flags1, 0, kChunks * 4);
    StatusBlock st0{}, st1{};
    std::thread producer([&]() {
      for (int c = 0; c < kChunks; ++c)
        iris_cpu_mp_produce(src.data() + c * kChunk / 4, sym(0, kA) + c * kChunk, kChunk, flags0 + c, 1, hb, 0, 1);
      for (int c = 0; c < kChunks; ++c) {  // then collect the doubled chunks from its own B
        const uint32_t s = iris_cpu_wait_flag(flags0 + c, 1, 1ull << 27, &st0, 0);
        CHECK(s == kOk, "producer wait chunk %d", c);
        memcpy(back.data() + c * kChunk / 4, sym(0, kB) + c * kChunk, kChunk);
      }
    });
    std::thread consumer([&]() {
      std::vector<int32_t> tmp(kChunk / 4);
      for (int c = 0; c < kChunks; ++c) {
        const uint32_t s = iris_cpu_wait_flag(flags1 + c, 1, 1ull << 27, &st1, 1);
        CHECK(s == kOk, "consumer wait chunk %d", c);
        const int32_t* in = reinterpret_cast<const int32_t*>(sym(1, kA) + c * kChunk);
        for (size_t i = 0; i < tmp.size(); ++i) tmp[i] = 2 * in[i];
        iris_cpu_mp_produce(tmp.data(), sym(1, kB) + c * kChunk, kChunk, flags1 + c, 1, hb, 1, 0);
      }
    });
    producer.join();
    consumer.join();
    bool ok = true;
    for (size_t i = 0; i < src.size(); ++i) ok = ok && back[i] == 2 * src[i];
    CHECK(ok, "message passing: dst != 2 * src");
    CHECK(st0.code == kOk && st1.code == kOk, "status after message passing");
  }

  // ---- 4. a wait on a flag that nothing sets runs out and reports where ----
  {
    uint32_t* flag = reinterpret_cast<uint32_t*>(sym(0, kF)) + 100;
    *flag = 3;
    StatusBlock st{};
    const uint32_t s = iris_cpu_wait_flag(flag, 4, 10000, &st, 0);
    CHECK(s == kTimeout, "wait must time out");
    CHECK(st.code == kTimeout && st.value == 3 && st.aux == 4, "status block: code %u value %llu aux %llu", st.code,
          (unsigned long long)st.value, (unsigned long long)st.aux);
  }

  // ---- 5. checking pointer translation ----
  {
    StatusBlock st{};
    const uint64_t good = iris_cpu_translate_checked(hb[0] + 256, hb, kHeap, 0, kWorld, 1, &st);
    CHECK(good == hb[1] + 256 && st.code == kOk, "translate inside the heap");
    const uint64_t bad = iris_cpu_translate_checked(hb[0] + kHeap + 8, hb, kHeap, 0, kWorld, 1, &st);
    CHECK(bad == 0 && st.code == kBadPointer, "pointer past the heap: code %u", st.code);
    StatusBlock st2{};
    const uint64_t bad_rank = iris_cpu_translate_checked(hb[0], hb, kHeap, 0, kWorld, 5, &st2);
    CHECK(bad_rank == 0 && st2.code == kBadRank, "rank out of range: code %u", st2.code);
  }

  // ---- 6. the inbox protocol of the fused GEMM's pushed one-shot / reduce-scatter paths, with random delays ----
  // Every "rank" (a thread) writes its partial into its slot of EVERY rank's inbox with ordinary stores, releases it
  // with an increment of the destination's cumulative flag, waits until its own flag has seen all ranks, and sums the
  // slots.  Inboxes alternate by call parity and nothing is reset between calls.  A call starts with the entry
  // handshake: every rank tells every rank that it has entered call c, and nobody pushes before all have.  Without it
  // a rank that is one call ahead can raise a destination's cumulative flag to W * c while a slow rank's
  // contribution to call c is still missing there (this model, run without the handshake, shows exactly that as a
  // wrong sum).  Under the thread sanitizer a missing release / acquire is a reported race; the sums catch the rest.
  {
    constexpr int W = 4, kCalls = 40, kElems = 192;
    // one "heap" per rank inside segment 0: [flag, entry flags (64 B) | inbox parity 0: W slots | inbox parity 1: W slots]
    constexpr uint64_t kRankBytes = 64 + 2ull * W * kElems * 4;
    static_assert(W * kRankBytes <= (64 << 10), "fits the data area A");
    uint8_t* region = sym(0, kA);
    memset(region, 0, W * kRankBytes);
    uint64_t hbw[W];
    for (int r = 0; r < W; ++r) hbw[r] = (uint64_t)(region + r * kRankBytes);
    std::atomic<int> failures{0};
    auto body = [&](int rank) {
      unsigned seed = 1234u + 77u * rank;
      auto nap = [&]() {
        seed = seed * 1664525u + 1013904223u;
        if ((seed >> 28) < 5) std::this_thread::sleep_for(std::chrono::microseconds((seed >> 20) & 63));
      };
      uint32_t* my_flag = reinterpret_cast<uint32_t*>(hbw[rank]);
      int32_t* my_inbox = reinterpret_cast<int32_t*>(hbw[rank] + 64);
      uint32_t* my_entry = my_flag + 8;  // entry flag of rank q at [8 + q]
      for (int call = 1; call <= kCalls; ++call) {
        const int par = call & 1;
        for (int i = 0; i < W; ++i) signal_set(my_entry + rank, (uint32_t)call, rank, (rank + 1 + i) % W, hbw);
        nap();
        for (int q = 0; q < W; ++q) {
          StatusBlock st{};
          if (wait_until_ge(my_entry + q, (uint32_t)call, 1ull << 27, &st, 5, rank, q) != kOk) {
            ++failures;
            return;
          }
        }
        for (int i = 0; i < W; ++i) {  // peers first, own copy last, as the kernel does
          const int dst = (rank + 1 + i) % W;
          nap();
          int32_t* slot = translate(my_inbox, rank, dst, hbw) + (par * W + rank) * kElems;
          for (int e = 0; e < kElems; ++e) slot[e] = call * 1000 + rank * 10 + (e & 7);
          signal_add(my_flag, 1u, rank, dst, hbw);
        }
        nap();
        StatusBlock st{};
        if (wait_until_ge(my_flag, (uint32_t)(W * call), 1ull << 27, &st, 6, rank, call) != kOk) {
          ++failures;
          return;
        }
        for (int e = 0; e < kElems; ++e) {
          long sum = 0;
          for (int sl = 0; sl < W; ++sl) sum += my_inbox[(par * W + sl) * kElems + e];
          const long want = (long)W * call * 1000 + 10 * (W * (W - 1) / 2) + (long)W * (e & 7);
          if (sum != want) {
            ++failures;
            return;
          }
        }
        nap();
      }
    };
    std::vector<std::thread> ranks;
    for (int r = 0; r < W; ++r) ranks.emplace_back(body, r);
    for (auto& t : ranks) t.join();
    CHECK(failures.load() == 0, "inbox protocol: %d rank(s) saw a wrong sum or a time-out", failures.load());
  }

  // ---- 7. the all-scatter protocol: pushes into every rank's OUTPUT, entry handshake, arrival counter ----
  // Outputs are not double-buffered: the consumer of call c's output (here: the check) runs between the calls, and
  // a peer's pushes of call c + 1 must not land before it has finished.  The entry flag (written when a rank starts a
  // call, i.e. after it has consumed the previous output) is what the pushers wait for; the arrival counter tells a
  // rank that all pushes of the call have landed in its own output.
  {
    constexpr int W = 4, kCalls = 40, kCols = 64;  // output row per rank: W column blocks of kCols ints
    constexpr uint64_t kRankBytes = 128 + (uint64_t)W * kCols * 4;
    uint8_t* region = sym(1, kA);
    memset(region, 0, W * kRankBytes);
    uint64_t hbw[W];
    for (int r = 0; r < W; ++r) hbw[r] = (uint64_t)(region + r * kRankBytes);
    std::atomic<int> failures{0};
    auto body = [&](int rank) {
      unsigned seed = 99u + 31u * rank;
      auto nap = [&]() {
        seed = seed * 1664525u + 1013904223u;
        if ((seed >> 28) < 5) std::this_thread::sleep_for(std::chrono::microseconds((seed >> 20) & 63));
      };
      uint32_t* done = reinterpret_cast<uint32_t*>(hbw[rank]);       // [0] arrival counter
      uint32_t* entry = done + 8;                                      // [8 + q] entry flag of rank q
      int32_t* out = reinterpret_cast<int32_t*>(hbw[rank] + 128);
      for (int call = 1; call <= kCalls; ++call) {
        for (int i = 0; i < W; ++i) signal_set(entry + rank, (uint32_t)call, rank, (rank + 1 + i) % W, hbw);
        nap();
        for (int q = 0; q < W; ++q) {
          StatusBlock st{};
          if (wait_until_ge(entry + q, (uint32_t)call, 1ull << 27, &st, 7, rank, q) != kOk) {
            ++failures;
            return;
          }
        }
        for (int i = 0; i < W; ++i) {  // this rank's column block into every rank's output
          const int dst = (rank + 1 + i) % W;
          int32_t* blk = translate(out, rank, dst, hbw) + rank * kCols;
          for (int e = 0; e < kCols; ++e) blk[e] = call * 100 + rank;
          nap();
        }
        for (int i = 0; i < W; ++i) signal_add(done, 1u, rank, (rank + 1 + i) % W, hbw);
        StatusBlock st{};
        if (wait_until_ge(done, (uint32_t)(W * call), 1ull << 27, &st, 8, rank, call) != kOk) {
          ++failures;
          return;
        }
        nap();  // "kernel end"; the host now reads the output
        for (int q = 0; q < W; ++q)
          for (int e = 0; e < kCols; ++e)
            if (out[q * kCols + e] != call * 100 + q) {
              ++failures;
              return;
            }
      }
    };
    std::vector<std::thread> ranks;
    for (int r = 0; r < W; ++r) ranks.emplace_back(body, r);
    for (auto& t : ranks) t.join();
    CHECK(failures.load() == 0, "all-scatter protocol: %d rank(s) saw a wrong block or a time-out", failures.load());
  }

  // ---- 8. the two-shot protocol: partials stay home, one owner per tile pulls, sums and pushes the result ----
  // Partial buffers alternate by call parity; outputs are single.  Per call: entry handshake; every rank stores its
  // partial of every tile in its OWN memory and raises the tile's flag on the tile's owner; the owner waits for W
  // arrivals, reads the partial of every rank (remote reads), and writes the sum into the output of EVERY rank; an
  // arrival counter per rank tells it that all owners have delivered; then the rank consumes its output.  What must
  // hold: no partial is overwritten while an owner still reads it (two calls later, same parity), and no output is
  // overwritten while its rank still consumes the previous result.
  {
    constexpr int W = 4, kCalls = 30, kTiles = 8, kElems = 48;
    // per rank: [done counter, entry flags (64 B) | tile flags (64 B) | partial[2][tiles][elems] | out[tiles][elems]]
    constexpr uint64_t kPartial = 128, kOut = kPartial + 2ull * kTiles * kElems * 4;
    constexpr uint64_t kRankBytes = kOut + (uint64_t)kTiles * kElems * 4;
    static_assert(W * kRankBytes <= (64 << 10), "fits the data area B");
    uint8_t* region = sym(0, kB);
    memset(region, 0, W * kRankBytes);
    uint64_t hbw[W];
    for (int r = 0; r < W; ++r) hbw[r] = (uint64_t)(region + r * kRankBytes);
    std::atomic<int> failures{0};
    auto body = [&](int rank) {
      unsigned seed = 4242u + 13u * rank;
      auto nap = [&]() {
        seed = seed * 1664525u + 1013904223u;
        if ((seed >> 28) < 4) std::this_thread::sleep_for(std::chrono::microseconds((seed >> 20) & 63));
      };
      uint32_t* done = reinterpret_cast<uint32_t*>(hbw[rank]);
      uint32_t* entry = done + 8;
      uint32_t* tflag = reinterpret_cast<uint32_t*>(hbw[rank] + 64);
      int32_t* partial = reinterpret_cast<int32_t*>(hbw[rank] + kPartial);
      int32_t* out = reinterpret_cast<int32_t*>(hbw[rank] + kOut);
      auto fail = [&]() { ++failures; };
      for (int call = 1; call <= kCalls; ++call) {
        const int par = call & 1;
        for (int i = 0; i < W; ++i) signal_set(entry + rank, (uint32_t)call, rank, (rank + 1 + i) % W, hbw);
        for (int q = 0; q < W; ++q) {
          StatusBlock st{};
          if (wait_until_ge(entry + q, (uint32_t)call, 1ull << 27, &st, 9, rank, q) != kOk) return fail();
        }
        for (int t = 0; t < kTiles; ++t) {  // "epilogue": partial tile into own memory, flag on the owner
          int32_t* mine = partial + (par * kTiles + t) * kElems;
          for (int e = 0; e < kElems; ++e) mine[e] = call * 1000 + t * 10 + rank;
          signal_add(tflag + t, 1u, rank, t % W, hbw);
          nap();
        }
        for (int t = rank; t < kTiles; t += W) {  // "reducer": the tiles this rank owns
          StatusBlock st{};
          if (wait_until_ge(tflag + t, (uint32_t)(W * call), 1ull << 27, &st, 10, rank, t) != kOk) return fail();
          int32_t sum[kElems] = {0};
          for (int q = 0; q < W; ++q) {
            const int32_t* theirs = translate(partial, rank, q, hbw) + (par * kTiles + t) * kElems;
            for (int e = 0; e < kElems; ++e) sum[e] += theirs[e];
          }
          nap();
          for (int i = 0; i < W; ++i) {
            int32_t* dst = translate(out, rank, (rank + 1 + i) % W, hbw) + t * kElems;
            for (int e = 0; e < kElems; ++e) dst[e] = sum[e];
          }
        }
        for (int i = 0; i < W; ++i) signal_add(done, 1u, rank, (rank + 1 + i) % W, hbw);
        StatusBlock st{};
        if (wait_until_ge(done, (uint32_t)(W * call), 1ull << 27, &st, 11, rank, call) != kOk) return fail();
        nap();  // "kernel end"; the host consumes the output
        for (int t = 0; t < kTiles; ++t)
          for (int e = 0; e < kElems; ++e)
            if (out[t * kElems + e] != W * (call * 1000 + t * 10) + W * (W - 1) / 2) return fail();
      }
    };
    std::vector<std::thread> ranks;
    for (int r = 0; r < W; ++r) ranks.emplace_back(body, r);
    for (auto& t : ranks) t.join();
    CHECK(failures.load() == 0, "two-shot protocol: %d rank(s) saw a wrong sum or a time-out", failures.load());
  }

  // ---- 9. the all-gather prologue: every rank pushes its own rows into every peer's gathered buffer ----
  // The gathered buffer is single (not alternated by call parity) and the kernel has no end-of-call handshake: a rank
  // may start call c + 1 while a peer still reads the rows of call c.  What keeps that peer's rows intact is the wait
  // of the pushing side for the PEER's entry flag of call c + 1 (written when the peer starts that call, i.e. after it
  // has read everything of call c) before the first remote store.  Chunk flags are cumulative arrival counters.
  {
    constexpr int W = 4, kCalls = 40, kElems = 96;
    // per rank: [entry flags (64 B) | chunk flags (64 B) | gathered[W][kElems]]
    constexpr uint64_t kGath = 128;
    constexpr uint64_t kRankBytes = kGath + (uint64_t)W * kElems * 4;
    static_assert(W * kRankBytes <= (64 << 10), "fits the data area B");
    uint8_t* region = sym(0, kB);
    memset(region, 0, W * kRankBytes);
    uint64_t hbw[W];
    for (int r = 0; r < W; ++r) hbw[r] = (uint64_t)(region + r * kRankBytes);
    std::atomic<int> failures{0};
    auto body = [&](int rank) {
      unsigned seed = 777u + 17u * rank;
      auto nap = [&]() {
        seed = seed * 1664525u + 1013904223u;
        if ((seed >> 28) < 5) std::this_thread::sleep_for(std::chrono::microseconds((seed >> 20) & 63));
      };
      uint32_t* entry = reinterpret_cast<uint32_t*>(hbw[rank]);
      uint32_t* cflag = reinterpret_cast<uint32_t*>(hbw[rank] + 64);
      int32_t* gathered = reinterpret_cast<int32_t*>(hbw[rank] + kGath);
      auto fail = [&]() { ++failures; };
      for (int call = 1; call <= kCalls; ++call) {
        // "host": this call's own rows (stream-ordered after the previous call of this rank)
        for (int e = 0; e < kElems; ++e) gathered[rank * kElems + e] = call * 1000 + rank * 10 + (e & 3);
        // kernel start: entry flag to every rank
        for (int i = 0; i < W; ++i) signal_set(entry + rank, (uint32_t)call, rank, (rank + 1 + i) % W, hbw);
        nap();
        // communication warps: wait for the peer's entry, then push own rows and count the chunk on the peer
        for (int i = 0; i + 1 < W; ++i) {
          const int peer = (rank - 1 - i + 2 * W) % W;
          StatusBlock st{};
          if (wait_until_ge(entry + peer, (uint32_t)call, 1ull << 27, &st, 12, rank, peer) != kOk) return fail();
          int32_t* dst = translate(gathered, rank, peer, hbw) + rank * kElems;
          for (int e = 0; e < kElems; ++e) dst[e] = gathered[rank * kElems + e];
          signal_add(cflag + rank, 1u, rank, peer, hbw);
          nap();
        }
        // producer: rows of every source, own first; peers' rows after their chunk flag
        for (int sp = 0; sp < W; ++sp) {
          const int src = (rank + sp) % W;
          if (src != rank) {
            StatusBlock st{};
            if (wait_until_ge(cflag + src, (uint32_t)call, 1ull << 27, &st, 13, rank, src) != kOk) return fail();
          }
          nap();
          for (int e = 0; e < kElems; ++e)
            if (gathered[src * kElems + e] != call * 1000 + src * 10 + (e & 3)) return fail();
        }
      }
    };
    std::vector<std::thread> ranks;
    for (int r = 0; r < W; ++r) ranks.emplace_back(body, r);
    for (auto& t : ranks) t.join();
    CHECK(failures.load() == 0, "all-gather protocol: %d rank(s) read rows of another call or timed out", failures.load());
  }

  // ---- 10. stream-K inside one rank: parked pieces, finisher, call counter in "device" memory ----
  // Threads play the scheduling units of one launch and walk the kernel's own work iterator.  A piece that does not
  // hold a tile's first k-blocks parks its partial sum in the slot sk_unit_of assigns it and counts itself on the tile
  // (release); the unit with the first k-blocks, whose piece closes its range, waits (bounded, acquire) for the count,
  // puts it back to zero and adds the parked values.  Every unit reads the call number at the start of a launch; the
  // last unit to leave advances it.  Launches follow one another like kernels on a stream (join = kernel boundary).
  {
    using iris::gemm::kSkSlots;
    using iris::gemm::sk_unit_of;
    using iris::gemm::Work;
    using iris::gemm::WorkIter;
    constexpr int kUnits = 6, kTiles = 20, kKb = 7, kDp = 12, kLaunches = 25;   // 8 split tiles over 6 units
    constexpr int kSk = kTiles - kDp;
    struct State {
      std::atomic<uint32_t> cnt[kSk];
      int64_t ws[kSk][kSkSlots];
      int64_t out[kTiles];
      std::atomic<uint32_t> calls, left;
    };
    static State stt;
    for (auto& c : stt.cnt) c.store(0);
    stt.calls.store(0);
    stt.left.store(0);
    std::atomic<int> failures{0};
    auto value = [](uint32_t call, int tile, int kb) { return (int64_t)call * 100000 + tile * 100 + kb; };
    for (int launch = 1; launch <= kLaunches; ++launch) {
      memset(stt.out, 0, sizeof(stt.out));
      auto unit_body = [&](int unit) {
        unsigned seed = 4242u + 31u * unit + 7u * launch;
        auto nap = [&]() {
          seed = seed * 1664525u + 1013904223u;
          if ((seed >> 28) < 4) std::this_thread::sleep_for(std::chrono::microseconds((seed >> 20) & 31));
        };
        const uint32_t call = stt.calls.load(std::memory_order_relaxed) + 1u;   // ordered by the "kernel boundary"
        const long long S = (long long)kSk * kKb;
        WorkIter it(unit, kUnits, kTiles, kKb, kDp, kUnits, 1);
        Work w;
        while (it.next(w)) {
          int64_t acc = 0;
          for (int kb = w.kb0; kb < w.kb1; ++kb) acc += value(call, w.tile, kb);
          nap();
          if (w.kb0 == 0 && w.kb1 == kKb) {
            stt.out[w.tile] = acc;
            continue;
          }
          const int t = w.tile - kDp;
          const int head = sk_unit_of((long long)t * kKb, S, kUnits);
          if (w.kb0 > 0) {
            const int slot = unit - head - 1;
            if (slot < 0 || slot >= kSkSlots) { ++failures; return; }
            stt.ws[t][slot] = acc;
            stt.cnt[t].fetch_add(1u, std::memory_order_release);
          } else {
            const uint32_t need = (uint32_t)(sk_unit_of((long long)(t + 1) * kKb - 1, S, kUnits) - head);
            if (unit != head || need < 1 || need > (uint32_t)kSkSlots) { ++failures; return; }
            uint64_t polls = 0;
            while (stt.cnt[t].load(std::memory_order_acquire) < need)
              if (++polls > (1ull << 28)) { ++failures; return; }
            stt.cnt[t].store(0u, std::memory_order_relaxed);
            for (uint32_t s2 = 0; s2 < need; ++s2) acc += stt.ws[t][s2];
            stt.out[w.tile] = acc;
          }
        }
        if (stt.left.fetch_add(1u, std::memory_order_acq_rel) + 1u == call * (uint32_t)kUnits)
          stt.calls.store(call, std::memory_order_relaxed);
      };
      std::vector<std::thread> units;
      for (int u = 0; u < kUnits; ++u) units.emplace_back(unit_body, u);
      for (auto& t : units) t.join();
      for (int tile = 0; tile < kTiles; ++tile) {
        int64_t want = 0;
        for (int kb = 0; kb < kKb; ++kb) want += value((uint32_t)launch, tile, kb);
        if (stt.out[tile] != want) ++failures;
      }
      if (stt.calls.load() != (uint32_t)launch) ++failures;
      for (auto& c : stt.cnt)
        if (c.load() != 0) ++failures;
    }
    CHECK(failures.load() == 0, "stream-K protocol: %d wrong sums, slots out of range, counters off or time-outs", failures.load());
  }

  for (int r = 0; r < kWorld; ++r) {
    CHECK(iris_cpu_heap_unmap(base[r], kHeap) == 0, "unmap");
    CHECK(iris_cpu_heap_unlink(name[r]) == 0, "unlink");
  }
  if (g_fail == 0) printf("stress OK\n");
  return g_fail == 0 ? 0 : 1;
}
