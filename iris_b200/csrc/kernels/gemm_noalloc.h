/* gemm_noalloc.h — a GEMM entry point for callers that are not allowed to allocate device memory.
 *
 * This entry point has no counterpart in the reference.
 *
 * Who it is for: code that runs where a device allocation is forbidden or would stall everything else —
 * a plug-in called from inside another framework's stream-ordered step, a serving loop that has handed its
 * whole memory budget to a pool, a callback that runs while other work is in flight and must not trigger the
 * implicit device-wide synchronisation that cudaMalloc / cudaFree can cause.  Such callers can hand over
 * input and output buffers they already own, but they cannot provide (or size) the kernel's working memory.
 *
 * What it does: out[M, N] = a[M, K] * bt[N, K]^T in bf16 with fp32 accumulation, computed by the same tcgen05
 * kernel as the plan-based entry points in its flagged "partial tile -> scratch -> sum -> output" mode.  The
 * scratch (status record, per-tile flags, the bf16 partial matrix) lives in a file-scope device array that
 * is part of the library image: every GPU that loads the library keeps IRIS_GEMM_NOALLOC_SCRATCH_BYTES
 * (about 8 MB) reserved until the process exits, whether or not this function is ever called.
 *
 * Limits: M * N <= IRIS_GEMM_NOALLOC_MAX_ELEMS and at most IRIS_GEMM_NOALLOC_MAX_TILES output tiles of
 * 128 x 256; N and K multiples of 8; all three base addresses and row pitches multiples of 16 bytes; lda and ldb
 * at least K, ldo at least N and below 2^31.  Larger problems are rejected with a non-zero return code and a message
 * (iris_gemm_last_error()).
 *
 * It calls no cudaMalloc, cudaFree or any other allocating routine, on the device or through a library.
 *
 * First call on a device: looks up the device address of the scratch array (cudaGetSymbolAddress), reads the
 * SM count and raises the kernel's shared-memory limit.  Make that first call with the device current and
 * before starting any stream capture on that device.
 *
 * Sharing: every call on a device uses the same scratch, which still holds the previous call's contents; the
 * function clears the per-tile flags on `stream` before it launches.  Two calls whose kernels may overlap on
 * the GPU (different streams without an ordering between them) race on that scratch: order them.  The first
 * call on a device may come from several host threads at once; the set-up is done once, under a lock.
 *
 * Returns 0 on success; -1 bad argument, -2 problem larger than the built-in scratch, -3 CUDA error.
 * After the stream has finished, iris_gemm_noalloc_status() reports whether a bounded wait inside the kernel
 * expired (0 = clean).
 */
#pragma once
#include <stdint.h>

#define IRIS_GEMM_NOALLOC_MAX_ELEMS (4u * 1024u * 1024u)  /* M * N, i.e. 8 MB of bf16 partials */
#define IRIS_GEMM_NOALLOC_MAX_TILES 4096
#define IRIS_GEMM_NOALLOC_HEADER_BYTES (256 + (16 + IRIS_GEMM_NOALLOC_MAX_TILES) * 4 + 192)
#define IRIS_GEMM_NOALLOC_SCRATCH_BYTES (IRIS_GEMM_NOALLOC_HEADER_BYTES + IRIS_GEMM_NOALLOC_MAX_ELEMS * 2u)

#ifdef __cplusplus
extern "C" {
#endif

/* a: [M, K] bf16, row pitch lda elements; bt: [N, K] bf16, row pitch ldb; out: [M, N] bf16, row pitch ldo.
 * stream: a cudaStream_t (0 = the default stream).  All pointers are device pointers of the current device. */
int iris_gemm_noalloc(const void* a, int64_t lda, const void* bt, int64_t ldb, void* out, int64_t ldo, int M, int N,
                      int K, void* stream);

/* Synchronises the current device and returns the status code left in the scratch by the calls made since the
 * previous query (0 = none, 1 = a bounded wait expired), then clears the record.  Not needed on the fast path. */
int iris_gemm_noalloc_status(void);

#ifdef __cplusplus
}
#endif
