/* Allocation-free GEMM entry point of libcatcoc_b200.so.
 *
 * This entry point has no counterpart in the reference (whose examples allocate everything
 * with aclrtMalloc / shmem_malloc before each launch). It exists for callers that are not
 * allowed to allocate device memory themselves and cannot let a library do it for them:
 * plug-ins that run inside a host runtime which carved up the whole GPU at start-up and hands
 * out fixed buffers, and latency-critical loops whose owners forbid any allocator call (and
 * the implicit synchronisation it may bring) once the loop is running.
 *
 * The regular path (ops/gemm.py -> catcoc_pad2d + catcoc_fused_launch) copies an operand whose
 * row pitch is not a multiple of 16 bytes into a freshly allocated, TMA-legal buffer. This
 * variant does the same copy into a fixed scratch area that lives inside the library image
 * (a file-scope `static __device__` array), so it calls no cudaMalloc / cudaFree and no
 * allocating library routine.
 *
 * Rules of use:
 *   - The caller passes the operands and the output; nothing else is needed.
 *   - Limits: each padded operand (rows x padded row bytes) must fit
 *     CATCOC_NOALLOC_OPERAND_BYTES; larger problems are refused with CATCOC_E_TOO_LARGE and a
 *     message naming the limit. Every GPU that loads the library holds
 *     CATCOC_NOALLOC_SCRATCH_BYTES of device memory for this until the process exits.
 *   - The first call on a device resolves the scratch address (cudaGetSymbolAddress with that
 *     device current) and prepares the kernels. Make that first call before starting any
 *     stream capture on the device.
 *   - All calls share the one scratch area, which keeps whatever the previous call left in
 *     it. The function rewrites every byte it later reads (operands are re-copied, padding
 *     and the status words are re-zeroed on `stream`), so consecutive calls on one stream are
 *     safe. Calls whose GPU work may overlap (different streams, different host threads)
 *     race on the scratch and must be serialised by the caller.
 *   - The per-device table of resolved scratch addresses is filled without a lock: two host
 *     threads whose first calls on one device coincide both look the symbol up and store the
 *     same address, which is harmless. It does not make their GPU work safe to overlap.
 */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CATCOC_NOALLOC_OPERAND_BYTES (8u << 20)                      /* per padded operand   */
#define CATCOC_NOALLOC_SCRATCH_BYTES (2u * CATCOC_NOALLOC_OPERAND_BYTES + 256u) /* whole area */

/* out[M, N] = A @ B with fp32 (int32 for int8) accumulation, on `stream` (a cudaStream_t).
 *   a: stored [M, K] ([K, M] if trans_a) with leading dimension lda (elements), any pitch
 *   b: stored [K, N] ([N, K] if trans_b) with leading dimension ldb
 *   out: row-major [M, ldc]; in_fmt: CATCOC_IN_*; out_fmt: CATCOC_FMT_*
 * Returns 0, or a negative CATCOC_E_* code with catcoc_last_error() set. A kernel-side
 * failure (a pipeline wait that ran out of time) is reported by the status words; read them
 * with catcoc_matmul_noalloc_status after synchronising the stream. */
int catcoc_matmul_noalloc(const void* a, int64_t lda, const void* b, int64_t ldb, void* out,
                          int64_t ldc, int M, int N, int K, int in_fmt, int out_fmt, int trans_a,
                          int trans_b, void* stream);

/* Copies the 8 status words of the last call on the current device to `host_words`
 * (synchronous, no allocation). Word 0 is 0 when the kernel finished normally. */
int catcoc_matmul_noalloc_status(uint32_t* host_words);

#ifdef __cplusplus
}
#endif
