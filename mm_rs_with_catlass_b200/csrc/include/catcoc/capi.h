/* C ABI of libcatcoc_b200.so. Everything the Python layer (ctypes) and plain C/C++ callers use.
 *
 * Conventions: functions return 0 on success and a negative CATCOC_E_* code (or a positive
 * cudaError_t / CUresult passed through as -1000-code) on failure; catcoc_last_error() returns
 * a human-readable description of the most recent failure on the calling thread.
 *
 * The op entry points play the role of the reference's launcher functions
 * (examples/dynamic_tiling/include/launch_map.h:18-19, impl/kernel_fp16.cpp:22-86) and its
 * per-op __global__ wrappers (examples/00_matmul_allreduce/matmul_allreduce.cpp:50-169). */
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define CATCOC_MAX_WORLD 8

enum {
  CATCOC_OK = 0,
  CATCOC_E_BAD_ARG = -1,
  CATCOC_E_ALIGNMENT = -2,   /* operand base / leading dimension not 16-byte aligned for TMA */
  CATCOC_E_DRIVER = -3,
  CATCOC_E_UNSUPPORTED = -4,
  CATCOC_E_NOMEM = -5,
  CATCOC_E_IO = -6,
  CATCOC_E_TOO_LARGE = -7,
};

/* operand element formats */
enum { CATCOC_IN_F16 = 0, CATCOC_IN_BF16 = 1, CATCOC_IN_S8 = 2, CATCOC_IN_E4M3 = 3,
       CATCOC_IN_E5M2 = 4,
       CATCOC_IN_MXE4M3 = 5, CATCOC_IN_MXE5M2 = 6 /* block-scaled: UE8M0 scale per 32 K-elements (sfa / sfb) */ };
/* output / partial element formats (== catcoc::ElemFmt) */
enum { CATCOC_FMT_F16 = 0, CATCOC_FMT_BF16 = 1, CATCOC_FMT_F32 = 2, CATCOC_FMT_S32 = 3 };
/* op modes (== catcoc::FusedMode) */
enum { CATCOC_MODE_LOCAL = 0, CATCOC_MODE_RS = 1, CATCOC_MODE_AR = 2, CATCOC_MODE_AG = 3 };

/* Communication tiling. Field-for-field superset of the reference's CocTilingParams
 * (examples/dynamic_tiling/include/info.h:29-42); see tiling/config.py for the mapping. */
typedef struct CatcocTiling {
  int bn;          /* tile columns: 64, 128 or 256 (0 = default 256)                    */
  int swizzle;     /* tiles per column group of the raster (0 = default)                */
  int num_ctas;    /* persistent CTAs (0 = one per SM)                                   */
  int seg_dim;     /* all-reduce ownership split: 0 rows, 1 cols, -1 auto                */
  int use_multicast; /* all-reduce broadcast through the NVLS multicast alias if mapped  */
  int rounds;      /* owner work is spread over this many rounds (0 = default); reduce-scatter / all-reduce */
  int cta_pair;    /* 2: 256-row tiles on 2-CTA clusters (tcgen05 cta_group::2); else 1 CTA */
  int pull;        /* reduce-scatter / all-reduce: 1 = partial tiles stay in the local heap and the owner
                      sums them through the switch (multimem.ld_reduce); needs the multicast alias   */
  int comm_warps;  /* communication / reducer warps per CTA, 1..5 (0 = 5); all-gather and pull flavours */
  int push_tma;    /* push flavour: 1 = partial tiles go to their owners' slabs by TMA stores (stamps one tile
                      late), 0 = by 16-byte stores, -1 = CATCOC_PUSH_TMA decides (default off)            */
} CatcocTiling;

typedef struct CatcocOpArgs {
  int mode;                /* CATCOC_MODE_*                                              */
  int in_fmt;              /* CATCOC_IN_*                                                */
  int M, N, K;             /* output grid rows (all-gather: W * m), cols, local K        */
  int trans_a, trans_b;    /* storage: A is [K, M] if trans_a, B is [N, K] if trans_b    */
  const void* a; int64_t lda;   /* leading dimension (elements) of the stored matrix     */
  const void* b; int64_t ldb;
  void* out; int64_t ldc; int out_fmt;
  CatcocTiling tiling;

  /* distributed part (ignored when W <= 1 or mode == LOCAL) */
  int rank, W;
  int partial_fmt;                         /* format of tiles crossing NVLink            */
  void* stage[CATCOC_MAX_WORLD];           /* staging slabs, one base per rank           */
  int64_t stage_parity_bytes;              /* distance between the two parity halves of a staging region: a
                                              property of the buffer (>= catcoc_stage_bytes / 2, multiple of 1024) */
  uint32_t* arrive[CATCOC_MAX_WORLD];      /* arrival stamps                             */
  void* ar_out[CATCOC_MAX_WORLD];          /* all-reduce output (parity 0) on every rank */
  int64_t ar_out_parity_bytes;
  void* ar_out_mc;                         /* multicast alias or NULL                    */
  uint32_t* done[CATCOC_MAX_WORLD];
  uint32_t* done_mc;
  void* part;                              /* pull flavour: this rank's partial buffer (parity 0) ... */
  void* part_mc;                           /* ... and its multicast alias                */
  int64_t part_parity_bytes;
  void* gathered_mc;                       /* all-gather with use_multicast: aliases of gathered / gflags */
  uint32_t* gflags_mc;
  void* gathered[CATCOC_MAX_WORLD];        /* all-gather: gathered A (parity 0)          */
  int64_t gathered_parity_bytes;
  uint32_t* gflags[CATCOC_MAX_WORLD];
  int ag_m;                                /* all-gather: rows of one shard              */
  int ag_ld;                               /* all-gather: row pitch (elements) of the gathered buffer, >= K, 16-byte multiple */
  int ag_raw;                              /* all-gather: 1 = `a` may have any alignment and any pitch >= K (it is fetched by
                                              the communication warps, never by TMA); then W == 1 is allowed too: the padding
                                              prologue of a local GEMM (`gathered[0]` is the padded copy, an output)          */

  /* block-scaled fp8 (CATCOC_IN_MX*): scale factors packed in 512-byte blocks of 128 rows x 4
   * K-blocks (row r, K-block s at (r % 32) * 16 + (r / 32) * 4 + s), block (row_tile, k128) at
   * (row_tile * sf_k_blocks + k128) * 512; A must be stored [M, K] and B [N, K] */
  const void* sfa; const void* sfb; int sf_k_blocks;

  /* quantised epilogue */
  const float* scale_m; const float* scale_n; const int32_t* bias;

  /* affine epilogue (affine != 0): out = cast(alpha * acc + beta * c_src[row, col] + bias_f[col]);
   * c_src has the format and row indexing of `out` (it may be `out` itself), bias_f is fp32 [N] */
  int affine; float alpha; float beta;
  const void* c_src; int64_t ldc_src; const float* bias_f;
  int act;                                 /* activation on the finished values, in fp32: 0 none, 1 gelu (tanh form),
                                              2 silu, 3 relu; floating-point outputs only (local GEMM, all-gather GEMM) */

  /* Group walk (mode LOCAL only, num_groups > 0): one launch runs num_groups products that share
   * N and K. M counts the rows of the whole output; group g owns rows [end_{g-1}, end_g), read from
   * group_ends (device int32, cumulative) or, when that is NULL, g * group_rows. The stored
   * operands may be larger than one product: a_rows_total x a_k_total and b_n_total x b_k_total
   * (0 = M, K, N, K). Row r of group g reads A row r - g * g_a_row_back; K coordinates start at
   * g * g_a_k (A) and g * g_b_k (B); a B stored [N, K] starts at row g * g_b_row; the per-column
   * vectors (scale_n, bias, bias_f) of group g start at element g * g_nvec. */
  int num_groups; const int32_t* group_ends; int group_rows;
  int a_rows_total, a_k_total, b_n_total, b_k_total;
  int g_a_row_back, g_a_k, g_b_row, g_b_k, g_nvec;

  /* Extents of the buffers handed in above, for the bounds-checked build of the library (0 = unknown):
   * [0] stage bytes, [1] arrive words, [2] done words, [3] ar_out bytes, [4] gathered bytes,
   * [5] gflags words, [6] partial buffer bytes, [7] out bytes. The launcher also checks the tensor maps
   * it builds over these buffers against them in every build. */
  int64_t limit[8];
  uint32_t* epoch_ptr; uint32_t* cta_counter; uint32_t* status;
  uint64_t timeout_ns;
  int withhold_signals;
  unsigned long long* trace;               /* optional 16 x u64 cycle counters (see params.h), or NULL */
  uint32_t* events; uint32_t events_cap;   /* optional event ring (4 + 4 * events_cap words, see params.h), or NULL */
} CatcocOpArgs;

const char* catcoc_last_error(void);
int catcoc_version(void);
int catcoc_is_checked_build(void);   /* 1: device-side bounds checks compiled in (see FusedParams::limit) */

/* Launches the fused kernel on `stream` (a cudaStream_t). */
int catcoc_fused_launch(const CatcocOpArgs* args, void* stream);

/* Workspace sizes (bytes / words) for given problem + tiling, identical on every rank. */
int64_t catcoc_stage_bytes(int M, int N, int W, int seg_dim, int bn, int cta_pair, int partial_fmt);
int64_t catcoc_arrive_words(int M, int N, int W, int seg_dim, int bn, int cta_pair);
int64_t catcoc_done_words(int M, int N, int W, int seg_dim, int bn, int cta_pair);
int64_t catcoc_gather_flag_words(int m, int K, int W, int elt_bytes);
int catcoc_num_sms(int device);

/* ---- scheduler introspection (host-side replay of the device index math, for tests) ---- */
typedef struct CatcocTile {
  int seg, tile_in_seg, mi, ni, m0, n0, rows, cols;
} CatcocTile;
int catcoc_sched_total_tiles(int M, int N, int bm, int bn, int W, int seg_dim);
int catcoc_sched_get_tile(int M, int N, int bm, int bn, int W, int seg_dim, int first_seg,
                          int swizzle, int t, CatcocTile* out);
int catcoc_sched_get_tile_rounds(int M, int N, int bm, int bn, int W, int seg_dim, int first_seg,
                                 int swizzle, int rounds, int t, CatcocTile* out);
/* order: 0 rotated (segment after segment from first_seg), 1 interleaved (tile i of every segment, then
 * tile i + 1: pull flavours), 2 local first (segment first_seg, then the others interleaved: multicast all-gather) */
int catcoc_sched_get_tile_order(int M, int N, int bm, int bn, int W, int seg_dim, int first_seg,
                                int swizzle, int order, int t, CatcocTile* out);
/* Host replay of the group walk of a grouped / batched / split-K launch: writes up to max_tiles
 * tiles in launch order (seg = group) and returns the walk's tile count. `ends` is host memory
 * here (cumulative rows per group) or NULL for uniform groups of group_rows rows. */
int catcoc_group_walk_replay(int M, int N, int bm, int bn, int num_groups, const int32_t* ends,
                             int group_rows, int max_tiles, CatcocTile* out);

/* ---- CPU oracle (naive fp32 / int32 loops; see csrc/oracle/oracle.cpp) ---- */
int catcoc_oracle_matmul_f32(const float* a, const float* b, float* c, int M, int N, int K,
                             int trans_a, int trans_b);
int catcoc_oracle_quant_matmul(const int8_t* a, const int8_t* b, const int32_t* bias,
                               int32_t* acc, int M, int N, int K, int trans_a, int trans_b);
int catcoc_oracle_dequant(const int32_t* acc, const float* scale_m, const float* scale_n,
                          float* out, int M, int N);
int64_t catcoc_oracle_compare(const float* out, const float* golden, int64_t n, float rtol,
                              double* mean_rel_bias);
/* the rest of the catalogue: out = alpha op(A) op(B) + beta C + bias[col] (C, bias may be NULL) */
int catcoc_oracle_gemm(const float* a, const float* b, const float* c, const float* bias, float* out, int M, int N,
                       int K, int trans_a, int trans_b, float alpha, float beta);
/* y = alpha op(A) x + beta y_in, A row-major [rows, cols] */
int catcoc_oracle_gemv(const float* a, const float* x, const float* y_in, float* y, int rows, int cols, int trans,
                       float alpha, float beta);
int catcoc_oracle_batched_matmul(const float* a, const float* b, float* out, int batch, int M, int N, int K,
                                 int trans_a, int trans_b);
/* grouped along M: rows [ends[g-1], ends[g]) of A [M_total, K] times B[g] ([K, N] or, trans_b, [N, K]) */
int catcoc_oracle_grouped_matmul(const float* a, const float* b, const int32_t* ends, int groups, float* out,
                                 int M_total, int N, int K, int trans_b);
/* grouped along K: out[g] = A[:, ks of g] B[ks of g, :], A stored [K_total, M], B stored [K_total, N] */
int catcoc_oracle_grouped_matmul_slice_k(const float* a, const float* b, const int32_t* ends, int groups, float* out,
                                         int M, int N, int K_total);
/* int8 grouped products with dequantisation (scale_n [groups, N]; scale_m [M_total] resp. [groups, M]);
 * CATCOC_E_TOO_LARGE when an exact sum does not fit the device's int32 accumulator */
int catcoc_oracle_grouped_quant_matmul(const int8_t* a, const int8_t* b, const int32_t* ends, int groups,
                                       const float* scale_m, const float* scale_n, float* out, int M_total, int N,
                                       int K, int trans_b);
int catcoc_oracle_grouped_quant_matmul_slice_k(const int8_t* a, const int8_t* b, const int32_t* ends, int groups,
                                               const float* scale_m, const float* scale_n, float* out, int M, int N,
                                               int K_total);
/* independent problems packed back to back, mnk = 3 ints per problem */
int catcoc_oracle_group_gemm(int count, const int32_t* mnk, const float* alphas, const float* betas, const float* a,
                             const float* b, const float* c, float* out);

/* ---- symmetric heap (csrc/shmem/host.cu) ---- */
typedef struct CatcocHeap CatcocHeap;
int catcoc_heap_create(int device, int rank, int world, int64_t bytes, CatcocHeap** out);
int64_t catcoc_heap_bytes(const CatcocHeap* h);          /* rounded-up size per rank       */
int catcoc_heap_export_fd(CatcocHeap* h);                /* POSIX fd of the local handle   */
int catcoc_heap_import_peer(CatcocHeap* h, int peer, int fd);  /* map a peer's handle      */
void* catcoc_heap_base(const CatcocHeap* h, int peer);   /* address of rank `peer`'s heap  */
int catcoc_heap_multicast_supported(int device);
int catcoc_heap_mc_create(CatcocHeap* h);                /* rank 0: create + return fd     */
int catcoc_heap_mc_join(CatcocHeap* h, int fd);          /* all: import (fd<0: own) + add device */
int catcoc_heap_mc_bind(CatcocHeap* h);                  /* all, after every rank joined   */
void* catcoc_heap_mc_base(const CatcocHeap* h);          /* multicast alias or NULL        */
int catcoc_heap_destroy(CatcocHeap* h);
/* fd passing between local processes over an abstract unix socket */
/* (one datagram = one fd + a one-byte tag chosen by the sender, e.g. its rank) */
int catcoc_fd_send(const char* sock_name, int fd, int tag, int timeout_ms);
int catcoc_fd_recv_open(const char* sock_name);          /* returns listening socket       */
int catcoc_fd_recv(int listen_sock, int timeout_ms, int* tag);  /* returns received fd     */
int catcoc_fd_close(int fd);

/* ---- device primitive kernels (csrc/kernels/shmem_prims.cu), used by tests and the heap ---- */
typedef struct CatcocShmemCtx {
  int rank, W;
  void* base[CATCOC_MAX_WORLD];   /* heap base of every rank in this process's address space */
  void* mc_base;                  /* multicast alias or NULL */
  uint32_t* signal_off;           /* unused */
  int64_t barrier_off;            /* byte offset of the barrier stamp array in the heap */
  int64_t scratch_off;
} CatcocShmemCtx;
int catcoc_shmem_barrier_all(const CatcocShmemCtx* ctx, uint32_t epoch, uint64_t timeout_ns,
                             uint32_t* status, void* stream);
int catcoc_shmem_put(const CatcocShmemCtx* ctx, int peer, int64_t dst_off, const void* src,
                     int64_t bytes, int64_t signal_off, uint32_t signal_val, void* stream);
int catcoc_shmem_get(const CatcocShmemCtx* ctx, int peer, void* dst, int64_t src_off,
                     int64_t bytes, void* stream);
int catcoc_shmem_wait_until(const CatcocShmemCtx* ctx, int64_t signal_off, uint32_t value,
                            uint64_t timeout_ns, uint32_t* status, void* stream);
int catcoc_shmem_mc_broadcast(const CatcocShmemCtx* ctx, int64_t dst_off, const void* src,
                              int64_t bytes, void* stream);
int catcoc_shmem_mc_reduce_bf16(const CatcocShmemCtx* ctx, void* dst, int64_t src_off,
                                int64_t n_elems, void* stream);

int catcoc_shmem_put_blocks(void);  /* blocks a put launches: each adds signal_val once */
/* copy rows into a buffer whose pitch is TMA-legal, zero-filling the padding */
int catcoc_pad2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t rows,
                 int64_t row_bytes, void* stream);

/* out = cast(alpha * sum over `slices` fp32 partials [rows, cols] (slice s at parts + s * slice_elems)
 *            + beta * c_src + bias[cols]); finishes a split-K product */
int catcoc_splitk_reduce(const float* parts, int slices, int64_t slice_elems, int rows, int cols, void* out,
                         int64_t ldc, int out_fmt, float alpha, float beta, const void* c_src,
                         int64_t ldc_src, const float* bias, void* stream);
/* y = alpha * op(A) x + beta * y_in, A row-major [rows, cols] of fp16 / bf16 / fp32 (CATCOC_FMT_*),
 * op = transpose when `trans` (then x has `rows` and y `cols` elements and `workspace` must hold
 * catcoc_gemv_workspace_floats(rows, cols, 1) floats) */
int64_t catcoc_gemv_workspace_floats(int rows, int cols, int trans);
int catcoc_gemv(const void* A, int64_t lda, int fmt, int rows, int cols, int trans, const void* x, void* y,
                const void* y_in, float alpha, float beta, float* workspace, void* stream);

/* ---- split-K product + one-shot all-reduce (csrc/kernels/small_allreduce.cu) ----
 * out[out_rows, cols] (fp16 / bf16, pitch ldc) = rows [out_row0, out_row0 + out_rows) of the sum over ranks of
 * round(sum over `slices` fp32 planes [rows, cols] of this rank): all rows for an all-reduce, the rank's share for a
 * reduce-scatter. The
 * rounded local sum goes to heap offset part_off (the parity half of this launch's epoch, rows * cols * 2 bytes), the
 * stamps to catcoc_splitk_allreduce_flag_words(...) words at flags_off (zeroed once, never reset). cols and ldc must be
 * multiples of 8. epoch_ptr / cta_counter / status: the launch bookkeeping of the fused kernels (CatcocOpArgs). */
int64_t catcoc_splitk_allreduce_flag_words(int rows, int cols, int W);
int catcoc_splitk_allreduce(const CatcocShmemCtx* ctx, const float* parts, int slices, int64_t slice_elems, int rows,
                            int cols, int out_row0, int out_rows, void* out, int64_t ldc, int fmt, int64_t part_off,
                            int64_t flags_off,
                            int use_multicast, uint32_t* epoch_ptr, uint32_t* cta_counter, uint32_t* status,
                            uint64_t timeout_ns, void* stream);

/* All-gather of a small row-sharded activation (same file): this rank's shard [m rows of row_bytes bytes, pitch
 * shard_pitch_bytes] lands in rows [rank * m, (rank + 1) * m) of every rank's buffer at heap offset gathered_off (pitch
 * gathered_pitch_bytes; the parity half of this launch's epoch), and the call's kernel returns when all W shards have
 * arrived in this rank's buffer. Stamps: catcoc_small_allgather_flag_words(...) words at flags_off. */
int64_t catcoc_small_allgather_flag_words(int m, int64_t row_bytes, int W);
int catcoc_small_allgather(const CatcocShmemCtx* ctx, const void* shard, int64_t shard_pitch_bytes, int m, int64_t row_bytes,
                           int64_t gathered_off, int64_t gathered_pitch_bytes, int64_t flags_off, int use_multicast,
                           uint32_t* epoch_ptr, uint32_t* cta_counter, uint32_t* status, uint64_t timeout_ns, void* stream);

/* ---- flash attention forward (csrc/kernels/flash_attn.cu) ----
 * out[b, h, i, :] = softmax_j(scale * q[b, h, i, :] . k[b, g(h), j, :]) v[b, g(h), j, :] with q [B, Hq, Sq, D],
 * k / v [B, Hk, Sk, D] and out [B, Hq, Sq, D], all contiguous fp16 or bf16 (fmt = CATCOC_FMT_*), D = 64 or 128,
 * Hq a multiple of Hk (grouped-query heads share a key / value head). causal: key j is visible to query i when
 * j <= i + (Sk - Sq). `status`: 8 device words as for the GEMM kernels. */
int catcoc_flash_attention(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk, int Sq,
                           int Sk, int D, int fmt, int causal, float scale, uint32_t* status, uint64_t timeout_ns,
                           void* stream);

/* ---- multi-head latent attention, decode step over a paged cache (csrc/kernels/mla_decode.cu) ----
 * q_nope [T, H, 512], q_rope [T, H, 64] (T = B * q_len new tokens, q_len 1..4), latent cache [num_pages, 128, 512],
 * rotary cache [num_pages, 128, 64], block_table [B, max_pages] and kv_lens [B] (device int32), out [T, H, 512]; all
 * contiguous, fp16 or bf16. Keys are [latent, rotary] (576 wide), values the latent. causal: new token t does not see
 * the new tokens behind it. `splits` slices per sequence (flash decoding); more than one needs `workspace` of
 * catcoc_mla_workspace_bytes(...) bytes. `status`: 8 device words as for the GEMM kernels. */
int64_t catcoc_mla_workspace_bytes(int B, int q_len, int H, int splits);
int catcoc_mla_decode(const void* q_nope, const void* q_rope, const void* ckv, const void* krope, const int* block_table,
                      const int* kv_lens, void* out, void* workspace, int B, int q_len, int H, int num_pages,
                      int max_pages, int fmt, int causal, float scale, int splits, uint32_t* status,
                      uint64_t timeout_ns, void* stream);

#ifdef __cplusplus
}
#endif
