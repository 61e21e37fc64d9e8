// Kernel parameter block and enums shared by the fused kernels, their launchers and the C API.
#pragma once
#include <cstdint>
#include <cuda.h>
#include "catcoc/sched.h"

namespace catcoc {

constexpr int kMaxWorld = 8;

// What the epilogue / producer do around the GEMM tiles.
enum FusedMode : int {
  MODE_LOCAL = 0,  // plain GEMM: tile -> out
  MODE_RS = 1,     // matmul + reduce-scatter: push partial tile to its owner, owner sums
                   //   (pull flavour: partial tile stays local, the owner sums through the switch)
  MODE_AR = 2,     // matmul + all-reduce: as RS, then the owner broadcasts the reduced tile
  MODE_AG = 3,     // all-gather + matmul: comm warps push the A shard, producer waits per chunk
};

// Tensor-core flavour (template parameter of the kernel).
enum MmaKind : int {
  KIND_F16 = 0,  // fp16 / bf16 operands, fp32 accumulate   (tcgen05 kind::f16)
  KIND_I8 = 1,   // int8 operands, int32 accumulate          (tcgen05 kind::i8)
  KIND_F8 = 2,   // e4m3 / e5m2 operands, fp32 accumulate    (tcgen05 kind::f8f6f4)
  KIND_MX = 3,   // e4m3 / e5m2 with UE8M0 scales per 32 K    (tcgen05 kind::mxf8f6f4.block_scale)
};

// Element formats of outputs and of the partial tiles that cross NVLink.
enum ElemFmt : int { FMT_F16 = 0, FMT_BF16 = 1, FMT_F32 = 2, FMT_S32 = 3 };

CATCOC_HD int fmt_bytes(int fmt) { return (fmt == FMT_F16 || fmt == FMT_BF16) ? 2 : 4; }

// Compile-time epilogue variants of the kernel; a launch picks the leanest one that covers it.
enum EpiVariant {
  EPI_PLAIN = 0,    // convert and store (local GEMM, all-gather GEMM)
  EPI_REDUCE = 1,   // + owner-side fold of the peers' partial tiles, pushes and stamps (RS / AR)
  EPI_FULL = 2,     // + int32 bias, per-row / per-column scales, alpha / beta / C / fp32 bias
  EPI_PULL = 3,     // plain stores of partial tiles into the local heap + stamps; extra warps reduce the
                    // owned tiles through the switch (multimem.ld_reduce) and store / broadcast them
};

// Element-wise function on finished (owned) tiles, after scales / affine terms.
enum Activation : int { ACT_NONE = 0, ACT_GELU_TANH = 1, ACT_SILU = 2, ACT_RELU = 3 };

// Error codes written to status[0] by a kernel that gave up on a wait.
enum StatusCode : uint32_t {
  STATUS_OK = 0,
  STATUS_TIMEOUT_PIPELINE = 1,  // an intra-CTA mbarrier wait ran out of time
  STATUS_TIMEOUT_ARRIVE = 2,    // a peer's partial tile never arrived (RS / AR owner side)
  STATUS_TIMEOUT_DONE = 3,      // an owner's reduced tile never arrived (AR tail)
  STATUS_TIMEOUT_GATHER = 4,    // a peer's A chunk never arrived (AG producer)
  STATUS_TIMEOUT_BARRIER = 5,   // barrier_all / wait_until ran out of time
  STATUS_BAD_ARGUMENT = 6,
  STATUS_OUT_OF_RANGE = 7,      // checked build: an offset left its buffer (what = site, expected = limit, seen = offset)
};

// Buffers whose extents the checked build (-DCATCOC_CHECKED) knows; index into FusedParams::limit.
// Byte counts for data, word counts for stamp arrays, 0 = unknown (not checked).
enum LimitId : int {
  LIM_STAGE = 0, LIM_ARRIVE = 1, LIM_DONE = 2, LIM_AR_OUT = 3, LIM_GATHERED = 4, LIM_GFLAGS = 5, LIM_PART = 6,
  LIM_OUT = 7, LIM_COUNT = 8,
};
// Where a checked access sits (status word `what` of STATUS_OUT_OF_RANGE).
enum CheckSite : uint32_t {
  SITE_PUSH_SLAB = 1,      // partial tile -> owner's staging slab
  SITE_FOLD_SLAB = 2,      // owner reads the peers' slabs
  SITE_ARRIVE_POST = 3,    // arrival stamp written
  SITE_ARRIVE_POLL = 4,    // arrival stamp polled
  SITE_DONE_POST = 5,
  SITE_DONE_POLL = 6,
  SITE_AR_OUT = 7,         // reduced tile -> every rank's output
  SITE_GATHER_PUSH = 8,    // A shard -> gathered buffer
  SITE_GFLAG_POST = 9,
  SITE_GFLAG_POLL = 10,
  SITE_PART_STORE = 11,    // pull flavour: partial tile -> local partial buffer
  SITE_PART_REDUCE = 12,   // pull flavour: in-switch sum of the partial copies
  SITE_OUT_STORE = 13,     // final rows -> out
  SITE_TMEM = 14,          // accumulator columns
};

// Layout of the status block (uint32 words): [0] code, [1] rank, [2] what (tile / chunk id),
// [3] expected, [4] seen, [5] peer, [6] blockIdx, [7] reserved.
constexpr int kStatusWords = 8;

struct alignas(64) FusedParams {
  CUtensorMap tm_a;          // A operand (AG: this rank's shard)
  CUtensorMap tm_a_gath[2];  // AG: gathered A, one map per parity buffer
  CUtensorMap tm_b;
  CUtensorMap tm_out;  // `out` as [rows, N] with a 32-row x 128-byte box (valid when out_tma)
  // Rank r's staging region as one matrix [slots * BM rows, BN] of partial elements (slots are
  // contiguous and BN wide), same box; valid when stage_tma
  CUtensorMap tm_stage[kMaxWorld];

  TileSched sched;
  int K;
  int mode;
  int rank, W;

  // operand staging: K elements per pipeline stage and per MMA instruction; smem majors
  int bk, umma_k;
  int a_mn_major, b_mn_major;
  int a_3d, b_3d;   // M/N-contiguous operand fetched through a 3-D map {128 B, K, blocks}: one TMA per stage
  uint32_t idesc;

  // output (MODE_LOCAL / MODE_AG / RS own tiles): row-major [rows, ldc]
  void* out;
  int64_t ldc;
  int out_fmt;      // ElemFmt of `out`
  int out_vec_ok;   // 1 when 16-byte vector stores to `out` are aligned
  int out_tma;      // 1 when tm_out describes `out`: finished 32-row x 128-byte windows leave by TMA store
  int stage_tma;    // 1 when tm_stage[r] describes rank r's staging slabs: partial tiles are pushed by TMA store
  int64_t out_row_shift;  // subtracted from the tile's global row to index `out` (RS: seg begin)

  // partial tiles that cross NVLink
  int partial_fmt;               // ElemFmt of pushed partial tiles
  uint8_t* stage[kMaxWorld];     // per-rank staging base (peer-mapped), see sched.h
  int64_t stage_parity_bytes;    // distance between the two parity halves of every rank's staging region
  uint32_t* arrive[kMaxWorld];   // per-rank arrival stamps
  // Pull flavour of RS / AR (pull != 0, needs the multicast alias): every rank stores its partial
  // [M, N] into its own heap at the same symmetric offset; the owner of a tile reads the sum of all
  // ranks' copies with multimem.ld_reduce (fp32 accumulation in the switch).
  int pull;
  CUtensorMap tm_part[2];        // this rank's partial buffer as [M, ldp] per parity, 32-row x 128-byte box
  uint8_t* part_local;           // this rank's partial buffer, parity 0
  const uint8_t* part_mc;        // multicast alias of the same buffer
  int64_t part_parity_bytes;
  int64_t ldp;                   // elements per row of the partial buffer
  // all-reduce broadcast targets
  uint8_t* ar_out[kMaxWorld];    // per-rank parity-0 output base; parity 1 at + ar_out_parity_bytes
  int64_t ar_out_parity_bytes;
  uint8_t* ar_out_mc;            // multicast alias of the same buffer (null => per-peer stores)
  uint32_t* done[kMaxWorld];     // per-rank "reduced tile landed" stamps
  uint32_t* done_mc;

  // all-gather
  const uint8_t* a_local;        // this rank's shard, row-major [m, K]
  int64_t a_local_pitch;         // bytes
  uint8_t* gathered[kMaxWorld];  // per-rank gathered buffer base (parity 0)
  int64_t gathered_parity_bytes;
  int64_t gathered_pitch;        // bytes per row of the gathered buffer
  uint32_t* gflags[kMaxWorld];   // per-rank chunk stamps
  // Raw shard (ag_raw != 0): the shard may start at any element and have any row pitch, so TMA never reads
  // it. The communication warps fetch it in units of a_vec bytes (the largest power of two that divides
  // base address and pitch) and also copy this rank's own rows into its gathered buffer, from where the
  // producer loads the local tiles like the remote ones. With W == 1 this is the padding prologue of a
  // local GEMM whose A has a pitch TMA cannot take: pad and product in one launch.
  int ag_raw;
  int a_vec;                     // 16, 8, 4 or 2
  int64_t a_row_bytes;           // valid bytes per shard row (K elements)
  uint8_t* gathered_mc;          // multicast aliases: one multimem.st lands a piece of the shard (and its
  uint32_t* gflags_mc;           //   stamp) on every rank; null => one store per peer
  GatherPlan gp;
  int elt_bytes_a;

  // quantised epilogue (KIND_I8 / KIND_F8): out = cast(float(acc) * scale_m[row] * scale_n[col])
  const float* scale_m;   // per output row (token), indexed by the global row; may be null
  const float* scale_n;   // per output column (channel); may be null
  const int32_t* bias;    // int32 [N], added to every rank's accumulator; may be null

  // affine epilogue on finished (owned) tiles, after the dequantisation above; off when
  // `affine` is 0:  out = cast(alpha * acc + beta * c_src[row, col] + bias_f[col])
  int affine;
  float alpha, beta;
  const void* c_src;      // same element format and row indexing as `out`; may be null
  int64_t ldc_src;        // elements per row of c_src
  const float* bias_f;    // fp32 [N]; may be null
  // activation applied last, in fp32, before the single rounding to the output format (Activation)
  int act;

  // Group walk (MODE_LOCAL only; num_groups == 0: off). One launch covers several GEMMs that
  // share N and K: the output's rows [begin_g, end_g) belong to group g. It serves grouped
  // (ragged rows per group), batched (uniform rows) and split-K (group = K slice) products.
  int num_groups;
  const int32_t* group_ends;  // device: cumulative row count after each group; null = uniform
  int group_rows;             // uniform groups: rows of every group
  int g_a_row_back;           // A row of output row r of group g:  r - g * g_a_row_back
  int g_a_k;                  // K coordinate of A starts at  g * g_a_k
  int g_b_row;                // N coordinate of B (stored [N, K]) starts at  g * g_b_row
  int g_b_k;                  // K coordinate of B starts at  g * g_b_k
  int g_nvec;                 // scale_n / bias / bias_f of group g start at  g * g_nvec

  // block-scaled fp8: scale factors packed in 512-byte blocks of 128 rows x 4 K-blocks
  // (row r, K-block s at (r % 32) * 16 + (r / 32) * 4 + s); block (row_tile, k128) at
  // ((row_tile * sf_k_blocks) + k128) * 512
  const uint8_t* sfa;
  const uint8_t* sfb;
  int sf_k_blocks;

  // launch bookkeeping
  uint32_t* epoch_ptr;       // completed launches on this workspace (local memory)
  uint32_t* cta_counter;     // CTAs finished in this launch (local memory)
  uint32_t* status;          // kStatusWords words, host-visible
  int64_t limit[LIM_COUNT];  // extents of the buffers above for the checked build (see LimitId)
  uint64_t timeout_ns;
  int withhold_signals;      // test hook: this rank posts no arrival / done / chunk stamps
  // Optional per-launch cycle counters (summed over CTAs), null = off:
  // [0] producer waits on empty   [1] producer issue     [2] MMA waits on full
  // [3] MMA waits on acc_empty    [4] MMA issue          [5] epilogue waits on acc_full
  // [6] epilogue work             [7] epilogue waits on peers' stamps   [8] CTA lifetime
  // [9] epilogue publish / rest   [10] owner-side reduce
  // [11] epilogue TMEM loads      [12] convert + stage to shared         [13] flush to global / peers
  // [14] epilogue time on owned tiles (accumulator ready -> tile done)   [15] the same on pushed tiles
  unsigned long long* trace;
  // Optional event ring (null = off): word 0 of `events` is the write cursor, records of four 32-bit
  // words follow from word 4 on: {globaltimer low, globaltimer high, cta << 16 | role << 8 | phase, tile}.
  // One lane per role writes a record at the start and at the end of every tile (EventRole / EventPhase);
  // the host turns the ring into a Chrome trace (utils/trace.py).
  uint32_t* events;
  uint32_t events_cap;       // records the ring can hold
};

enum EventRole : uint32_t { EV_PRODUCER = 0, EV_MMA = 1, EV_EPILOGUE = 2, EV_COMM = 3, EV_REDUCER = 4 };
enum EventPhase : uint32_t { EV_BEGIN = 0, EV_END = 1, EV_WAIT_PEER = 2 };

}  // namespace catcoc
