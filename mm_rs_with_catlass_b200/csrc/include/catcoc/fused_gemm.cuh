// The one persistent, warp-specialised sm_100a kernel behind every op of this library.
//
//   warp 0      TMA producer A : cp.async.bulk.tensor K-slices of A -> 128B-swizzled smem ring
//                                (all-gather: waits for the peers' chunk stamps first)
//   warp 1      MMA issuer     : one elected lane issues tcgen05.mma into a double-buffered TMEM
//                                accumulator, tcgen05.commit frees smem stages / publishes tiles
//   warps 2..5  epilogue       : tcgen05.ld -> convert (bias / dequant / alpha, beta / activation in the
//                                fuller variants) -> smem staging -> one TMA store per window for local
//                                outputs, coalesced 16 B stores to a peer's staging slab (NVLink P2P) or to
//                                every rank's output (P2P or multimem.st); in the push flavour owner tiles
//                                fold the peers' partials into the fp32 / int32 accumulator first, in the
//                                pull flavour every tile is stored locally and its owner is stamped
//   warp 6      TMA producer B : K-slices of B into the same ring (one warp cannot issue both
//                                operands' copies fast enough)
//   warps 7..11 (384-thread variants; warp 7 alone in the 256-thread ones)
//               communication  : all-gather: send this rank's A shard, peer by peer or once by multimem.st
//                                (raw shards of any pitch; with one rank this is the padding prologue);
//               reducers       : pull flavour: wait for a tile's W stamps, read the sum of all ranks' partials
//                                through the switch (multimem.ld_reduce), store it or broadcast it + done stamp
//
// The collective is expressed inside the tile loop (see sched.h for the visiting order), so
// transfers overlap the tensor-core work tile by tile and no NCCL call is involved.
//
// Cross-GPU synchronisation uses epoch stamps: a producer writes the launch's epoch number into
// a per-(tile, source) word with st.release.sys after its data; a consumer polls with
// ld.acquire.sys until the stamp reaches the epoch. Stamps are never reset, staging buffers are
// double-buffered by epoch parity, and every wait is bounded (status word + clean return).
//
// Roles of the reference this kernel replaces (different construction, same jobs):
//   include/catcoc/dgemm/kernel/matmul_allreduce.hpp:114-313
//   include/catcoc/dgemm/kernel/allgather_matmul.hpp:108-263
//   include/catcoc/dgemm/kernel/matmul_reduce_scatter.hpp:107-298
//   include/catcoc/dgemm/kernel/quant_matmul_reduce_scatter.hpp:116-351
//   3rdparty/catlass/include/catlass/gemm/block/block_mmad_pingpong.hpp:181-319
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "catcoc/params.h"
#include "catcoc/ptx.cuh"

namespace catcoc {

constexpr int kBM = 128;               // rows per CTA == TMEM lanes
constexpr int kMaxBN = 256;            // tile cols upper bound == TMEM columns per accumulator
constexpr int kABytes = kBM * 128;     // A stage: 128 rows x 128 B (K-major) or the MN-major equal
constexpr int kEpiWarps = 4;
constexpr int kEpiWinBytes = 32 * 128;             // one staged window: 32 rows x 128 B
constexpr int kEpiStageBytes = 2 * kEpiWinBytes;   // per epilogue warp: two windows (one may still feed a TMA store)
constexpr int kThreads = 256;          // warps 0-6 are the GEMM roles, warp 7 a communication warp
// The plain-epilogue variant (the only one the all-gather runs) fits 204 registers per thread, so
// it carries two more communication warps: the push of the A shard is latency bound per warp and
// one warp per SM could not feed the link (measured 173 GB/s per GPU, the GEMM waited on it).
constexpr int kThreadsPlain = 384;
CATCOC_HD constexpr int threads_for(int epi) { return (epi == EPI_PLAIN || epi == EPI_PULL) ? kThreadsPlain : kThreads; }
constexpr int kTmemCols = 512;
constexpr int kPullStrips = 4;   // pull flavour: a 32-row quarter is reduced in this many strips (one reducer task each)
constexpr int kMaxStages = 6;

// Two flavours of the same kernel:
//   single : one CTA per 128 x bn tile, B stage = bn rows            (48 KiB / stage, 4 stages)
//   pair   : a 2-CTA cluster per 256 x bn tile (tcgen05 cta_group::2). Each CTA loads its own
//            128 rows of A and HALF of the B tile; the pair's leader issues one MMA that reads
//            both halves, so operand traffic into shared memory per FLOP halves
//                                                                     (32 KiB / stage, 6 stages)
// A pipeline stage holds kKPS consecutive K-blocks (each: A block + B block). Handing a stage
// from the producers to the MMA warp and back costs a few hundred cycles of barrier / commit
// latency that does not depend on how many MMAs the stage feeds, so the pair flavour (32 KiB per
// K-block) packs two K-blocks per stage: 8 MMAs per hand-off instead of 4, same bytes in flight.
#ifndef CATCOC_KPS_PAIR
#define CATCOC_KPS_PAIR 2
#endif
#ifndef CATCOC_KPS_SINGLE
#define CATCOC_KPS_SINGLE 1
#endif
template <bool CTA2> struct Geo {
  static constexpr int kKPS = CTA2 ? CATCOC_KPS_PAIR : CATCOC_KPS_SINGLE;
  static constexpr int kBBytesMax = (CTA2 ? kMaxBN / 2 : kMaxBN) * 128;
  static constexpr int kSubBytes = kABytes + kBBytesMax;        // one K-block: A then B
  static constexpr int kStageBytes = kKPS * kSubBytes;
  static constexpr int kStages = (192 * 1024) / kStageBytes;
  static constexpr int kSmemBytes =
      kStages * kStageBytes + kEpiWarps * kEpiStageBytes + 256 /*barriers*/ + 1024 /*align slack*/;
};

struct SmemTail {
  uint64_t full[kMaxStages];
  uint64_t empty[kMaxStages];
  uint64_t acc_full[2];
  uint64_t acc_empty[2];
  uint32_t tmem_base;
  uint32_t abort_flag;
  uint32_t dead;   // the status block already held an error when this CTA started
};

CATCOC_DEVICE void report_status(const FusedParams& p, uint32_t code, uint32_t what,
                                 uint32_t expected, uint32_t seen, uint32_t peer) {
  if (p.status == nullptr) return;
  if (atomicCAS(p.status, 0u, code) == 0u) {
    p.status[1] = static_cast<uint32_t>(p.rank);
    p.status[2] = what;
    p.status[3] = expected;
    p.status[4] = seen;
    p.status[5] = peer;
    p.status[6] = blockIdx.x;
    __threadfence_system();
  }
}

// Bounds-checked build (-DCATCOC_CHECKED): every offset into a workspace, a peer's memory, the
// output or the accumulator goes through CATCOC_BOUND(p, site, end, limit_id): `end` is one past
// the last byte (word, column) the access touches. An offset outside its buffer is recorded once
// in the status block (site, limit, offset) and the access is SKIPPED, so a wrong index shows up
// as an error with a location instead of as a fault or as wrong numbers somewhere else. In the
// normal build the macro is the constant `true` and costs nothing.
#if defined(CATCOC_CHECKED)
CATCOC_DEVICE bool bound_ok(const FusedParams& p, uint32_t site, int64_t end, int64_t limit) {
  if (limit <= 0 || (end >= 0 && end <= limit)) return true;   // 0: the caller did not tell the extent
  report_status(p, STATUS_OUT_OF_RANGE, site, static_cast<uint32_t>(limit), static_cast<uint32_t>(end),
                static_cast<uint32_t>(static_cast<uint64_t>(end) >> 32));
  return false;
}
#define CATCOC_BOUND(p, site, end, id) ::catcoc::bound_ok((p), (site), static_cast<int64_t>(end), (p).limit[(id)])
#define CATCOC_BOUND_ABS(p, site, end, lim) ::catcoc::bound_ok((p), (site), static_cast<int64_t>(end), static_cast<int64_t>(lim))
#else
#define CATCOC_BOUND(p, site, end, id) (true)
#define CATCOC_BOUND_ABS(p, site, end, lim) (true)
#endif

// One record of the optional event ring (see FusedParams::events); call from ONE lane of a role.
// Compiled into the diagnostic build only (-DCATCOC_CHECKED, loaded with CATCOC_CHECKED=1): in the
// register-capped 384-thread variants even the dormant call cost spills in the epilogue.
CATCOC_DEVICE void emit_event(const FusedParams& p, uint32_t role, uint32_t phase, uint32_t tile) {
#if !defined(CATCOC_CHECKED)
  (void)p; (void)role; (void)phase; (void)tile;
  return;
#endif
  if (p.events == nullptr) return;
  const uint32_t slot = atomicAdd(p.events, 1u);
  if (slot >= p.events_cap) return;
  const uint64_t t = ptx::globaltimer_ns();
  uint32_t* r = p.events + 4 + 4 * static_cast<size_t>(slot);
  r[0] = static_cast<uint32_t>(t);
  r[1] = static_cast<uint32_t>(t >> 32);
  r[2] = (blockIdx.x << 16) | (role << 8) | phase;
  r[3] = tile;
}

// Cycle accounting for the optional trace counters.
struct Tick {
  long long t;
  bool on;
  CATCOC_DEVICE explicit Tick(bool enabled) : t(enabled ? ptx::clock_cycles() : 0), on(enabled) {}
  CATCOC_DEVICE void lap(unsigned long long& acc) {
    if (on) { const long long n = ptx::clock_cycles(); acc += static_cast<unsigned long long>(n - t); t = n; }
  }
};

// Polls a stamp until it reaches `epoch` (wrap-safe), the time budget ends or the CTA aborts.
// `pace_ns` > 0 sleeps that long between polls (for waits that are expected to be long and must
// not load the memory system meanwhile).
CATCOC_DEVICE bool wait_stamp(const uint32_t* flag, uint32_t epoch, uint64_t timeout_ns,
                              volatile uint32_t* abort_flag, uint32_t* seen, uint32_t pace_ns = 0) {
  uint32_t v = ptx::ld_acquire_sys_u32(flag);
  if (static_cast<int32_t>(v - epoch) >= 0) return true;
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    if (pace_ns) __nanosleep(pace_ns);
    v = ptx::ld_acquire_sys_u32(flag);
    if (static_cast<int32_t>(v - epoch) >= 0) return true;
    if ((++spins & 0xf) == 0) {
      if (*abort_flag || ptx::globaltimer_ns() - t0 > timeout_ns) {
        *seen = v;
        return false;
      }
      __nanosleep(64);
    }
  }
}

// ---- value conversion helpers ---------------------------------------------------------
CATCOC_DEVICE uint32_t pack2(float a, float b, int fmt) {
  if (fmt == FMT_BF16) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
  }
  __half2 h = __floats2half2_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
CATCOC_DEVICE float2 unpack2(uint32_t u, int fmt) {
  if (fmt == FMT_BF16) {
    __nv_bfloat162 h = *reinterpret_cast<__nv_bfloat162*>(&u);
    return __bfloat1622float2(h);
  }
  __half2 h = *reinterpret_cast<__half2*>(&u);
  return __half22float2(h);
}

// activation on a finished value (fp32 in, fp32 out)
CATCOC_DEVICE float activate(float x, int act) {
  if (act == ACT_GELU_TANH) {
    // 0.5 x (1 + tanh(sqrt(2/pi) (x + 0.044715 x^3))), hardware tanh approximation (about 2^-11 relative)
    const float u = 0.7978845608028654f * x * (1.0f + 0.044715f * x * x);
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(u));
    return 0.5f * x * (1.0f + t);
  }
  if (act == ACT_SILU) return x / (1.0f + __expf(-x));
  if (act == ACT_RELU) return fmaxf(x, 0.0f);
  return x;
}

// 16 bytes from an address that is only `vec`-byte aligned (vec = 8, 4 or 2), of which the first
// `valid` (even, possibly <= 0) hold data; the rest reads as zero and is never touched in memory.
CATCOC_DEVICE uint4 load16_pieces(const uint8_t* src, int vec, int valid) {
  uint32_t w[4] = {0u, 0u, 0u, 0u};
  int b = 0;
  if (vec >= 8) {
    for (; b + 8 <= valid; b += 8) {
      const uint2 v = *reinterpret_cast<const uint2*>(src + b);
      w[b >> 2] = v.x;
      w[(b >> 2) + 1] = v.y;
    }
  }
  if (vec >= 4) {
    for (; b + 4 <= valid; b += 4) w[b >> 2] = *reinterpret_cast<const uint32_t*>(src + b);
  }
  for (; b + 2 <= valid; b += 2)
    w[b >> 2] |= static_cast<uint32_t>(*reinterpret_cast<const uint16_t*>(src + b)) << ((b & 2) * 8);
  return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- epilogue staging -----------------------------------------------------------------
// Each epilogue warp owns a 32 x 128 B staging area. Thread `lane` (one tile row) writes
// 16-byte units at a position XOR-swizzled with the row so that neither the row-wise writes
// nor the unit-wise reads conflict on banks.
CATCOC_DEVICE void stage_write(uint32_t stg, int lane, int unit, uint4 v) {
  ptx::st_shared_v4(stg + lane * 128 + ((unit ^ (lane & 7)) << 4), v);
}

// Writes the staged 32 x 128 B block out. Lanes cooperate so that 8 lanes cover one 128-byte
// row segment. `cols_valid` counts elements of `elt` bytes inside the matrix within this
// 128-byte window; `rows_valid` in [0, 32]. Destinations:
//   mc != nullptr          : one multimem.st per unit reaches every rank (aligned tiles only)
//   peer_bases != nullptr  : the same block goes to peer_bases[rank], [rank+1], ... (+ off)
//   otherwise              : `base` only
CATCOC_DEVICE void flush_staged(uint32_t stg, int lane, uint8_t* base, int64_t pitch,
                                int rows_valid, int cols_valid, int elt, bool vec_ok,
                                uint8_t* mc, uint8_t* const* peer_bases, int64_t off, int rank,
                                int W) {
  const int unit = lane & 7;
  const int per_unit = 16 / elt;
  const int c0 = unit * per_unit;
  const int ndst = (peer_bases != nullptr) ? W : 1;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    const int row = it * 4 + (lane >> 3);
    const uint4 v = ptx::ld_shared_v4(stg + row * 128 + ((unit ^ (row & 7)) << 4));
    if (row < rows_valid && c0 < cols_valid) {
      const int64_t rel = row * pitch + unit * 16;
      const bool full = vec_ok && (c0 + per_unit <= cols_valid);
      if (mc != nullptr) {
        ptx::multimem_st_v4(mc + rel, v);
      } else {
        for (int d = 0; d < ndst; ++d) {
          uint8_t* ptr = (peer_bases != nullptr)
                             ? peer_bases[peer_for_push_rs(rank, d, W)] + off + rel
                             : base + rel;
          if (full) {
            ptx::st_global_v4(ptr, v);
          } else {
            const int n = min(per_unit, cols_valid - c0);
            const uint32_t w[4] = {v.x, v.y, v.z, v.w};
            if (elt == 2) {
              for (int e = 0; e < n; ++e)
                *reinterpret_cast<uint16_t*>(ptr + e * 2) =
                    static_cast<uint16_t>(w[e >> 1] >> ((e & 1) * 16));
            } else {
              for (int e = 0; e < n; ++e) *reinterpret_cast<uint32_t*>(ptr + e * 4) = w[e];
            }
          }
        }
      }
    }
  }
}

// ---------------------------------------------------------------------------------------
// Group walk: one launch over several products that share N and K (grouped, batched, split-K).
// The tile list is the concatenation of the groups' tile grids, rows fastest inside a group, so
// that the CTAs working side by side share the group's B columns. Group extents live in device
// memory (a routing result need not visit the host), so every warp derives the tile count and
// walks the list with a cursor that only moves forward.
// ---------------------------------------------------------------------------------------
// called by a converged warp; every lane gets the sum
CATCOC_DEVICE int grouped_total_tiles(const FusedParams& p, int lane) {
  const int nt = ceil_div(p.sched.N, p.sched.BN);
  int sum = 0;
  for (int g = lane; g < p.num_groups; g += 32) {
    const int b = (g == 0) ? 0 : group_end_row(p.group_ends, p.group_rows, p.sched.M, g - 1);
    sum += ceil_div(max(0, group_end_row(p.group_ends, p.group_rows, p.sched.M, g) - b), p.sched.BM) * nt;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
  return sum;
}

CATCOC_DEVICE GroupWalk group_walk_begin(const FusedParams& p) {
  return group_walk_begin(p.num_groups, p.group_ends, p.group_rows, p.sched.M);
}

// `t` must be below the total and must not decrease between calls on the same cursor
CATCOC_DEVICE TileInfo walk_tile(const FusedParams& p, int t, GroupWalk& w) {
  if (p.num_groups == 0) return get_tile(p.sched, t);
  return group_walk_tile(p.sched, p.num_groups, p.group_ends, p.group_rows, t, w);
}

// ---------------------------------------------------------------------------------------
// The kernel
// ---------------------------------------------------------------------------------------
template <int KIND, bool CTA2, int EPI>
__global__ void __launch_bounds__(threads_for(EPI), 1)
fused_gemm_kernel(const __grid_constant__ FusedParams p) {
  // Epilogue variant (see EpiVariant in params.h): stages a launch cannot need are compiled out.
  constexpr bool kReduce = (EPI == EPI_REDUCE || EPI == EPI_FULL);   // push flavour of RS / AR: peers' partials, pushes, stamps
  constexpr bool kScale = (EPI == EPI_FULL);      // int32 bias, dequantisation, alpha / beta / C / fp32 bias
  constexpr bool kPull = (EPI == EPI_PULL);       // pull flavour of RS / AR: local partials, stamps, reducer warps
  using G = Geo<CTA2>;
  constexpr int kStages = G::kStages;
  constexpr int kStageBytes = G::kStageBytes;
  constexpr int kSubBytes = G::kSubBytes;
  constexpr int kKPS = G::kKPS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>(
      (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* epi_stage = smem + kStages * kStageBytes;
  SmemTail* tail = reinterpret_cast<SmemTail*>(epi_stage + kEpiWarps * kEpiStageBytes);
  volatile uint32_t* abort_flag = &tail->abort_flag;

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const TileSched& sched = p.sched;
  const int BN = sched.BN;
  // K-blocks per stage at run time: narrow single-CTA tiles (bn <= 64, the small-M configs) leave
  // room for two 24 KiB K-blocks in a 48 KiB stage, which halves their barrier hand-offs too.
  const int kps = (!CTA2 && BN <= 64) ? 2 : kKPS;
  const int sub_bytes = (kps != kKPS) ? (kABytes + BN * 128) : kSubBytes;
  const int num_kb = ceil_div(p.K, p.bk * kps);   // pipeline stages per tile
  // (a raw-shard all-gather runs on one rank too: the padding prologue of a local GEMM)
  const bool fused = (p.mode != MODE_LOCAL) && (p.W > 1 || (p.mode == MODE_AG && p.ag_raw != 0));
  const bool pull = kPull && fused && (p.pull != 0) && (p.mode == MODE_RS || p.mode == MODE_AR);
  // Pair flavour: `sub` is this CTA's half of the 256-row tile, work is dealt out per pair.
  const int sub = CTA2 ? static_cast<int>(ptx::cluster_ctarank()) : 0;
  const bool leader = (sub == 0);
  const int worker = CTA2 ? static_cast<int>(blockIdx.x >> 1) : static_cast<int>(blockIdx.x);
  const int num_workers = CTA2 ? static_cast<int>(gridDim.x >> 1) : static_cast<int>(gridDim.x);
  const int b_cols_cta = CTA2 ? BN / 2 : BN;   // columns of the B tile this CTA loads
  const uint32_t b_stage_bytes = static_cast<uint32_t>(b_cols_cta) * 128u;
  const int qpt = sched.BM / 32;               // 32-row quarters per tile: 4 (single) or 8 (pair)
  // TMEM columns: two accumulators at 0 and acc_stride. The block-scaled kind runs 128-column
  // tiles so that columns [256, 288) stay free for the scale factors of two stages in flight.
  const uint32_t acc_stride = (KIND == KIND_MX) ? 128u : static_cast<uint32_t>(kMaxBN);
  constexpr uint32_t kSfTmemCol = 256;         // + slot * 16: SFA 4 columns, SFB 4 columns per 128 of N
  constexpr int kSfSmemOff = kABytes + 128 * 128;   // inside a 48 KiB stage, after A and a 128-column B
  const bool grouped = (p.num_groups > 0);
  const int total_tiles = grouped ? grouped_total_tiles(p, lane) : sched.total_tiles;

  if (threadIdx.x == 0) {
    for (int s = 0; s < kStages; ++s) {
      ptx::mbar_init(&tail->full[s], 2);   // A-producer warp + B-producer warp
      ptx::mbar_init(&tail->empty[s], 1);
    }
    for (int b = 0; b < 2; ++b) {
      ptx::mbar_init(&tail->acc_full[b], 1);
      ptx::mbar_init(&tail->acc_empty[b], CTA2 ? 2 * kEpiWarps : kEpiWarps);
    }
    tail->abort_flag = 0;
    // A fused launch that finds an earlier failure latched in the status block does nothing: the
    // ranks' epochs no longer agree, so every wait would only run into its time limit again.
    tail->dead = (p.mode != MODE_LOCAL && (p.W > 1 || (p.mode == MODE_AG && p.ag_raw != 0)) &&
                  ptx::ld_relaxed_sys_u32(p.status) != 0u) ? 1u : 0u;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&p.tm_a);
    ptx::prefetch_tmap(&p.tm_b);
    if (p.out_tma) ptx::prefetch_tmap(kPull && p.pull ? &p.tm_part[0] : &p.tm_out);
  }
  if (warp == 1) {
    if (CTA2) {
      ptx::tmem_alloc_pair(&tail->tmem_base, kTmemCols);
      ptx::tmem_relinquish_pair();
    } else {
      ptx::tmem_alloc(&tail->tmem_base, kTmemCols);
      ptx::tmem_relinquish();
    }
  }
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (CTA2) ptx::cluster_sync_all();   // the peer's barriers exist before anyone signals them
  ptx::tcgen05_fence_after();
  const uint32_t tmem_base = tail->tmem_base;
  // both CTAs of a pair must take the same decision (they meet again at cluster barriers)
  bool dead = tail->dead != 0u;
  if (CTA2) dead = dead || ptx::ld_shared_cluster_u32(ptx::map_to_cta(ptx::smem_u32(&tail->dead), static_cast<uint32_t>(sub ^ 1))) != 0u;
  const long long cta_t0 = (p.trace != nullptr) ? ptx::clock_cycles() : 0;

  // Epoch of this launch: completed launches + 1. Read before any CTA can finish.
  uint32_t epoch = 1;
  if (fused) epoch = ptx::ld_relaxed_sys_u32(p.epoch_ptr) + 1;
  const int parity = static_cast<int>(epoch & 1u);

  if (dead) {
    // nothing to do: fall through to the teardown
  } else if (warp == 0) {
    // =============================== TMA producer ===============================
    int stage = 0;
    uint32_t phase = 0;
    uint32_t issued_mask = 0, issued_parity = 0;
    bool ok = true;
    const bool tr = (p.trace != nullptr) && lane == 0;
    unsigned long long c_wait = 0, c_issue = 0;
    Tick tick(tr);
    bool pre_ok = false, pre_valid = false;   // all-gather: stamps of the next tile sampled early
    int pre_tile = -1;
    GroupWalk walk = group_walk_begin(p);
    for (int t = worker; ok && t < total_tiles; t += num_workers) {
      const TileInfo ti = walk_tile(p, t, walk);
      const CUtensorMap* tma = &p.tm_a;
      int a_row = ti.m0 + sub * kBM;
      int a_k_off = 0;
      if (grouped) {
        a_row -= ti.seg * p.g_a_row_back;
        a_k_off = ti.seg * p.g_a_k;
      }
      if (p.mode == MODE_AG && fused) {
        if (ti.seg == p.rank && p.ag_raw == 0) {
          a_row = ti.mi * sched.BM + sub * kBM;  // row inside the local shard
        } else {
          // Every K-slice of this row chunk of source `seg` must have landed here. The stamps
          // were sampled (relaxed, non-blocking) while the previous tile was streaming; only
          // if that sample was too early does the warp fall back to a blocking poll.
          const uint32_t* fl = p.gflags[p.rank];
          bool ready = pre_valid && pre_tile == t && __all_sync(0xffffffffu, pre_ok);
          if (!ready) {
            for (int s = lane; ok && s < p.gp.n_slices; s += 32) {
              uint32_t seen = 0;
              const int64_t idx = gather_flag_index(p.gp, ti.seg, ti.mi, s);
              if (!CATCOC_BOUND(p, SITE_GFLAG_POLL, idx + 1, LIM_GFLAGS)) continue;
              if (!wait_stamp(fl + idx, epoch, p.timeout_ns, abort_flag, &seen)) {
                report_status(p, STATUS_TIMEOUT_GATHER, static_cast<uint32_t>(idx), epoch, seen,
                              static_cast<uint32_t>(ti.seg));
                *abort_flag = 1;
                ok = false;
              }
            }
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          } else {
            ptx::fence_acq_rel_sys();   // relaxed sample + fence = acquire
            __syncwarp();
          }
          ptx::fence_proxy_async();  // peer-written rows are about to be read by TMA
          tma = &p.tm_a_gath[parity];
        }
        // sample the stamps of the next remote tile now; the answer is needed one tile later
        pre_valid = false;
        const int tn = t + num_workers;
        if (tn < sched.total_tiles) {
          const TileInfo tin = get_tile(sched, tn);
          if (tin.seg != p.rank || p.ag_raw != 0) {
            const uint32_t* fl = p.gflags[p.rank];
            bool okl = true;
            for (int s = lane; s < p.gp.n_slices; s += 32) {
              const int64_t fi = gather_flag_index(p.gp, tin.seg, tin.mi, s);
              if (!CATCOC_BOUND(p, SITE_GFLAG_POLL, fi + 1, LIM_GFLAGS)) { okl = false; continue; }
              const uint32_t v = ptx::ld_relaxed_sys_u32(fl + fi);
              okl = okl && (static_cast<int32_t>(v - epoch) >= 0);
            }
            pre_ok = okl;
            pre_valid = true;
            pre_tile = tn;
          }
        }
      }
      if (lane == 0) emit_event(p, EV_PRODUCER, EV_BEGIN, static_cast<uint32_t>(t));
      for (int kb = 0; kb < num_kb; ++kb) {
        tick.lap(c_issue);
        const bool got = ptx::mbar_wait(&tail->empty[stage], phase ^ 1u, p.timeout_ns, abort_flag);
        tick.lap(c_wait);
        if (!got) {
          if (lane == 0) {
            report_status(p, STATUS_TIMEOUT_PIPELINE, 0u, static_cast<uint32_t>(t),
                          static_cast<uint32_t>(kb), 0u);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        if (ptx::elect_one()) {
          const int per_box = 128 / p.elt_bytes_a;
          const uint32_t bar = CTA2 ? ptx::map_to_cta(ptx::smem_u32(&tail->full[stage]), 0u) : 0u;
          // Single flavour: this warp arms its own barrier with its bytes. Pair flavour: both
          // CTAs' copies are credited to the leader's barrier and only the leader arms it, with
          // the bytes of the whole pair. K-blocks past the end of K are fetched as zeros.
          if (KIND == KIND_MX) {
            // A block + the 512-byte scale-factor block of (this 128-row tile, this K-block)
            ptx::mbar_expect_tx(&tail->full[stage], kABytes + 512);
            const int row_tile = a_row / kBM;
            ptx::bulk_load_1d(smem + stage * kStageBytes + kSfSmemOff,
                              p.sfa + (static_cast<int64_t>(row_tile) * p.sf_k_blocks + kb) * 512, 512,
                              &tail->full[stage]);
          } else if (!CTA2) ptx::mbar_expect_tx(&tail->full[stage], kps * kABytes);
          else if (leader) ptx::mbar_expect_tx(&tail->full[stage], 2u * kps * kABytes);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (j >= kps) break;
            uint8_t* sa = smem + stage * kStageBytes + j * sub_bytes;
            const int k0 = (kb * kps + j) * p.bk + a_k_off;
            if (!CTA2) {
              if (!p.a_mn_major) {
                ptx::tma_load_2d(sa, tma, &tail->full[stage], k0, a_row);
              } else if (p.a_3d) {
                ptx::tma_load_3d(sa, tma, &tail->full[stage], 0, k0, a_row / per_box);
              } else {
                // storage [K, M]: boxes of 128 B along M x bk rows of K
                for (int b = 0; b < kBM / per_box; ++b)
                  ptx::tma_load_2d(sa + b * (p.bk * 128), tma, &tail->full[stage], a_row + b * per_box, k0);
              }
            } else {
              if (!p.a_mn_major) {
                ptx::tma_load_2d_pair(sa, tma, bar, k0, a_row);
              } else if (p.a_3d) {
                ptx::tma_load_3d_pair(sa, tma, bar, 0, k0, a_row / per_box);
              } else {
                for (int b = 0; b < kBM / per_box; ++b)
                  ptx::tma_load_2d_pair(sa + b * (p.bk * 128), tma, bar, a_row + b * per_box, k0);
              }
            }
          }
        }
        __syncwarp();
        issued_mask |= 1u << stage;
        issued_parity = (issued_parity & ~(1u << stage)) | (phase << stage);
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
    if (tr) { atomicAdd(p.trace + 0, c_wait); atomicAdd(p.trace + 1, c_issue); }
    if (*abort_flag && lane == 0 && leader) {
      // let every bulk copy this thread started land before the CTA's smem goes away
      volatile uint32_t never = 0;
      for (int s = 0; s < kStages; ++s)
        if (issued_mask & (1u << s))
          ptx::mbar_wait(&tail->full[s], (issued_parity >> s) & 1u, 2000000ull, &never);
    }
  } else if (warp == 1) {
    // =============================== MMA issuer ===============================
    // The whole warp walks the loop converged (so addresses and descriptors stay warp-uniform
    // and cheap); one elected lane issues the tcgen05 instructions.
    if (leader) {
      int stage = 0;
      uint32_t phase = 0;
      int acc = 0;
      uint32_t acc_phase = 0;
      bool ok = true;
      const uint32_t a_lbo = p.a_mn_major ? static_cast<uint32_t>(p.bk) * 128u : 16u;
      const uint32_t b_lbo = p.b_mn_major ? static_cast<uint32_t>(p.bk) * 128u : 16u;
      // descriptor low-word increment per MMA along K (units of 16 bytes)
      const uint32_t a_kinc = (p.a_mn_major ? static_cast<uint32_t>(p.umma_k) * 128u : 32u) >> 4;
      const uint32_t b_kinc = (p.b_mn_major ? static_cast<uint32_t>(p.umma_k) * 128u : 32u) >> 4;
      const uint32_t stage_inc = static_cast<uint32_t>(kStageBytes) >> 4;
      const uint64_t da0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem), a_lbo, 1024u);
      const uint64_t db0 = ptx::make_smem_desc_sw128(ptx::smem_u32(smem) + kABytes, b_lbo, 1024u);
      const uint32_t idesc = p.idesc;
      const int k_per_stage = p.bk / p.umma_k;   // 4
      const int umma_k = p.umma_k;
      const int K = p.K;
      const bool tr = (p.trace != nullptr) && lane == 0;
      unsigned long long c_full = 0, c_acc = 0, c_issue = 0;
      Tick tick(tr);
      bool probed = false;
      for (int t = worker; ok && t < total_tiles; t += num_workers) {
        tick.lap(c_issue);
        const bool got_acc = ptx::mbar_wait(&tail->acc_empty[acc], acc_phase ^ 1u, p.timeout_ns, abort_flag);
        tick.lap(c_acc);
        if (!got_acc) {
          if (lane == 0) {
            report_status(p, STATUS_TIMEOUT_PIPELINE, 1u, static_cast<uint32_t>(t), 0u, 0u);
            *abort_flag = 1;
          }
          break;
        }
        ptx::tcgen05_fence_after();
        if (lane == 0) emit_event(p, EV_MMA, EV_BEGIN, static_cast<uint32_t>(t));
        const uint32_t tmem_d = tmem_base + static_cast<uint32_t>(acc) * acc_stride;
        for (int kb = 0; kb < num_kb; ++kb) {
          tick.lap(c_issue);
          // `probed` is the answer of a non-blocking probe issued before the previous stage's
          // MMAs: its latency was hidden behind their issue, so a ready stage costs nothing here
          const bool got_full = probed || ptx::mbar_wait(&tail->full[stage], phase, p.timeout_ns, abort_flag);
          tick.lap(c_full);
          if (!got_full) {
            if (lane == 0) {
              report_status(p, STATUS_TIMEOUT_PIPELINE, 2u, static_cast<uint32_t>(t),
                            static_cast<uint32_t>(kb), 0u);
              *abort_flag = 1;
            }
            ok = false;
            break;
          }
          ptx::tcgen05_fence_after();
          // K tail: TMA zero-fills beyond K, MMAs entirely out of range are skipped.
          const int k_mmas = ceil_div(K, umma_k);                    // MMAs along K for a whole tile
          const int k_first = kb * kps * k_per_stage;                // index of this stage's first MMA
          const uint64_t da = da0 + static_cast<uint64_t>(stage * stage_inc);
          const uint64_t db = db0 + static_cast<uint64_t>(stage * stage_inc);
          {
            const int ns = (stage + 1 == kStages) ? 0 : stage + 1;
            const uint32_t np = (stage + 1 == kStages) ? (phase ^ 1u) : phase;
            probed = ptx::mbar_test_wait(&tail->full[ns], np);
          }
          if (KIND == KIND_MX) {
            if (ptx::elect_one()) {
              // scale factors of this stage: shared -> TMEM (slot alternates with the stage so a
              // copy never overwrites columns an earlier, still running MMA may read)
              const uint32_t sf_smem = ptx::smem_u32(smem + stage * kStageBytes + kSfSmemOff);
              const uint32_t sf_tmem = tmem_base + kSfTmemCol + static_cast<uint32_t>(stage & 1) * 16u;
              const int nblk = BN / 128;
              ptx::tmem_cp_32x128b_warpx4(sf_tmem, ptx::make_smem_desc_noswizzle(sf_smem, 128u, 128u));
              for (int j = 0; j < nblk; ++j)
                ptx::tmem_cp_32x128b_warpx4(sf_tmem + 4u * (1 + j),
                                            ptx::make_smem_desc_noswizzle(sf_smem + 512u * (1 + j), 128u, 128u));
#pragma unroll
              for (int k = 0; k < 4; ++k) {
                if (k_first + k < k_mmas) {
                  const uint64_t dak = da + static_cast<uint64_t>(k * a_kinc);
                  const uint64_t dbk = db + static_cast<uint64_t>(k * b_kinc);
                  const uint32_t accum = (k_first + k) != 0 ? 1u : 0u;
                  // K-block k of the four in a scale word: byte k, passed both as the id in the
                  // descriptor and in the top bits of the scale addresses
                  const uint32_t sel = static_cast<uint32_t>(k) << 30;
                  ptx::umma_mxf8(tmem_d, dak, dbk, ptx::with_sf_ids(idesc, k, k), (sf_tmem) | sel,
                                 (sf_tmem + 4u) | sel, accum);
                }
              }
              ptx::tcgen05_commit(&tail->empty[stage]);
              if (kb == num_kb - 1) ptx::tcgen05_commit(&tail->acc_full[acc]);
            }
          } else if (ptx::elect_one()) {
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const int j = kk >> 2, k = kk & 3;
              if (j < kps && k_first + kk < k_mmas) {
                const uint64_t dak = da + static_cast<uint64_t>(j * (sub_bytes >> 4) + k * a_kinc);
                const uint64_t dbk = db + static_cast<uint64_t>(j * (sub_bytes >> 4) + k * b_kinc);
                const uint32_t accum = (k_first + kk) != 0 ? 1u : 0u;
                if (CTA2) {
                  if (KIND == KIND_F16) ptx::umma_f16_pair(tmem_d, dak, dbk, idesc, accum);
                  else if (KIND == KIND_I8) ptx::umma_i8_pair(tmem_d, dak, dbk, idesc, accum);
                  else ptx::umma_f8f6f4_pair(tmem_d, dak, dbk, idesc, accum);
                } else {
                  if (KIND == KIND_F16) ptx::umma_f16(tmem_d, dak, dbk, idesc, accum);
                  else if (KIND == KIND_I8) ptx::umma_i8(tmem_d, dak, dbk, idesc, accum);
                  else if (KIND == KIND_F8) ptx::umma_f8f6f4(tmem_d, dak, dbk, idesc, accum);
                }
              }
            }
            // frees this smem stage (in both CTAs of a pair) once the MMAs above retire
            if (CTA2) ptx::tcgen05_commit_pair(&tail->empty[stage], 3);
            else ptx::tcgen05_commit(&tail->empty[stage]);
            if (kb == num_kb - 1) {
              if (CTA2) ptx::tcgen05_commit_pair(&tail->acc_full[acc], 3);
              else ptx::tcgen05_commit(&tail->acc_full[acc]);
            }
          }
          __syncwarp();
          if (++stage == kStages) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        if (lane == 0) emit_event(p, EV_MMA, EV_END, static_cast<uint32_t>(t));
        acc ^= 1;
        if (acc == 0) acc_phase ^= 1u;
      }
      tick.lap(c_issue);
      if (tr) { atomicAdd(p.trace + 2, c_full); atomicAdd(p.trace + 3, c_acc); atomicAdd(p.trace + 4, c_issue); }
      if (*abort_flag && lane == 0) {
        // wait (bounded) for the tensor core to retire what was issued before TMEM is freed
        volatile uint32_t never = 0;
        if (CTA2) ptx::tcgen05_commit_pair(&tail->acc_full[acc], 3);
        else ptx::tcgen05_commit(&tail->acc_full[acc]);
        ptx::mbar_wait(&tail->acc_full[acc], acc_phase, 2000000ull, &never);
      }
    }
  } else if (warp < 2 + kEpiWarps) {
    // =============================== epilogue ===============================
    // The four epilogue warps never synchronise with each other: warp q owns tile rows
    // [32q, 32q+32) end to end, including their stamps, so a warp that gives up on a wait
    // cannot strand the others at a barrier.
    const int q = warp & 3;                 // TMEM lane quarter this warp may read
    const uint32_t stg_base = ptx::smem_u32(epi_stage + (warp - 2) * kEpiStageBytes);
    uint32_t win_count = 0;   // windows staged so far: picks the staging buffer
    const int row_base = sub * kBM + q * 32;   // first tile row of this warp
    const int row_in_tile = row_base + lane;
    const int qid = sub * 4 + q;               // quarter index inside the tile
    const bool is_int = (KIND == KIND_I8);
    const bool dequant = kScale && ((p.scale_m != nullptr) || (p.scale_n != nullptr));
    const int pfmt = p.partial_fmt;
    const int pelt = fmt_bytes(pfmt);
    int acc = 0;
    uint32_t acc_phase = 0;
    bool ok = true;
    const bool tr = (p.trace != nullptr) && lane == 0 && q == 0;
    unsigned long long c_full = 0, c_work = 0, c_peer = 0, c_pub = 0, c_own = 0;
    unsigned long long c_tld = 0, c_cvt = 0, c_flush = 0, c_tile_own = 0, c_tile_push = 0;
    Tick tick(tr);
    // A partial tile pushed by TMA store is announced one tile late: the arrival stamp may only
    // follow the completion of the tile's bulk stores, and waiting for that right away would
    // stall the warp for a link round trip. `pending_stamp` is the stamp still owed (lane 0).
    const bool any_tma = (p.out_tma != 0) || (kReduce && p.stage_tma != 0);
    uint32_t* pending_stamp = nullptr;
    bool prev_win_tma = false;   // the most recent window of this warp left by a TMA store
    auto settle_pending = [&]() {
      // every bulk store of this warp is complete; its stamp can go out
      if (lane == 0 && pending_stamp != nullptr) {
        ptx::bulk_wait_group_all();
        ptx::fence_proxy_async();
        ptx::st_release_sys_u32(pending_stamp, epoch);
      }
      pending_stamp = nullptr;
    };

    GroupWalk walk = group_walk_begin(p);
    for (int t = worker; ok && t < total_tiles; t += num_workers) {
      const TileInfo ti = walk_tile(p, t, walk);
      const bool own = !kReduce || !fused || (p.mode == MODE_AG) || (ti.seg == p.rank);
      const bool reduce_here = kReduce && fused && own && (p.mode == MODE_RS || p.mode == MODE_AR);
      const int st_fmt = (own && !pull) ? p.out_fmt : pfmt;   // format of what this tile's epilogue stores
      const int st_elt = fmt_bytes(st_fmt);
      const int rows_valid = max(0, min(32, ti.rows - row_base));
      const int nvec_off = grouped ? ti.seg * p.g_nvec : 0;   // this group's per-column vectors
      const bool affine = kScale && (p.affine != 0) && own;

      tick.lap(c_work);
      if (reduce_here) {
        // never wait on a peer while owing one a stamp
        if (kReduce) settle_pending();
        // the peers' rows [32q, 32q+32) of this tile must have landed in my staging slabs
        if (lane < p.W && lane != p.rank) {
          uint32_t seen = 0;
          const int64_t idx = arrive_flag_index(sched, ti.tile_in_seg, lane) * qpt + qid;
          if (!CATCOC_BOUND(p, SITE_ARRIVE_POLL, idx + 1, LIM_ARRIVE)) {
            ok = false;
          } else if (!wait_stamp(p.arrive[p.rank] + idx, epoch, p.timeout_ns, abort_flag, &seen)) {
            report_status(p, STATUS_TIMEOUT_ARRIVE, static_cast<uint32_t>(ti.tile_in_seg), epoch,
                          seen, static_cast<uint32_t>(lane));
            *abort_flag = 1;
            ok = false;
          }
        }
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
      }

      tick.lap(c_peer);
      const bool got_tile = ptx::mbar_wait(&tail->acc_full[acc], acc_phase, p.timeout_ns, abort_flag);
      tick.lap(c_full);
      if (!got_tile) {
        if (lane == 0) {
          report_status(p, STATUS_TIMEOUT_PIPELINE, 3u, static_cast<uint32_t>(t), 0u, 0u);
          *abort_flag = 1;
        }
        break;
      }
      ptx::tcgen05_fence_after();
      if (lane == 0 && q == 0) emit_event(p, EV_EPILOGUE, EV_BEGIN, static_cast<uint32_t>(t));
      const long long tile_t0 = tr ? ptx::clock_cycles() : 0;
      const uint32_t taddr =
          tmem_base + (static_cast<uint32_t>(q * 32) << 16) + static_cast<uint32_t>(acc) * acc_stride;

      // Where this warp's 32 rows of the tile go.
      uint8_t* base = nullptr;           // single destination
      int64_t pitch = 0;
      uint8_t* mc = nullptr;             // multicast destination
      uint8_t* const* peer_bases = nullptr;  // broadcast by per-peer stores
      int64_t off = 0;
      bool vec_ok = true;
      const int64_t row_shift = pull ? 0 : p.out_row_shift;
      if (kPull && pull) {
        // the partial tile goes to its true (m, n) position of this rank's own partial buffer
        pitch = p.ldp * st_elt;
        base = p.part_local + static_cast<int64_t>(parity) * p.part_parity_bytes +
               (static_cast<int64_t>(ti.m0 + row_base) * p.ldp + ti.n0) * st_elt;
        vec_ok = (p.out_vec_ok != 0) && ((ti.n0 * st_elt) % 16 == 0);
      } else if (!own) {
        pitch = static_cast<int64_t>(BN) * st_elt;
        base = p.stage[ti.seg] + stage_slot_offset(sched, st_elt, p.stage_parity_bytes, parity, p.rank, ti.tile_in_seg) +
               static_cast<int64_t>(row_base) * pitch;
      } else if (kReduce && fused && p.mode == MODE_AR) {
        pitch = p.ldc * st_elt;
        off = static_cast<int64_t>(parity) * p.ar_out_parity_bytes +
              (static_cast<int64_t>(ti.m0 + row_base) * p.ldc + ti.n0) * st_elt;
        vec_ok = (p.out_vec_ok != 0) && ((ti.n0 * st_elt) % 16 == 0);
        if (p.ar_out_mc != nullptr && vec_ok && (ti.cols % (16 / st_elt) == 0)) {
          mc = p.ar_out_mc + off;
        } else {
          peer_bases = p.ar_out;
        }
      } else {
        pitch = p.ldc * st_elt;
        base = static_cast<uint8_t*>(p.out) +
               (static_cast<int64_t>(ti.m0 + row_base - row_shift) * p.ldc + ti.n0) * st_elt;
        vec_ok = (p.out_vec_ok != 0) && ((ti.n0 * st_elt) % 16 == 0);
      }

      // checked build: the last byte this warp stores for this tile must lie inside its buffer
      bool dst_ok = true;
#if defined(CATCOC_CHECKED)
      if (rows_valid > 0 && ti.cols > 0) {
        const int64_t span = static_cast<int64_t>(rows_valid - 1) * pitch + static_cast<int64_t>(ti.cols) * st_elt;
        if (kPull && pull) {
          dst_ok = CATCOC_BOUND(p, SITE_PART_STORE, (base - p.part_local) + span, LIM_PART);
        } else if (!own) {   // slabs are stored whole
          dst_ok = CATCOC_BOUND(p, SITE_PUSH_SLAB, (base - p.stage[ti.seg]) + 31 * pitch + static_cast<int64_t>(BN) * st_elt,
                                LIM_STAGE);
        } else if (kReduce && fused && p.mode == MODE_AR) {
          dst_ok = CATCOC_BOUND(p, SITE_AR_OUT, off + span, LIM_AR_OUT);
        } else {
          dst_ok = CATCOC_BOUND(p, SITE_OUT_STORE, (base - static_cast<uint8_t*>(p.out)) + span, LIM_OUT);
        }
      }
#endif

      const int groups = BN / 32;                        // 32-column groups in the accumulator
      const int groups_per_win = (st_elt == 2) ? 2 : 1;  // groups per 128 B window of output
      const int nwin = groups / groups_per_win;
      const int last_group = min(groups, ceil_div(ti.cols, 32)) - 1;
      bool released = false;

      // Finished windows of a local output leave through the TMA store unit (one instruction
      // per 4 KiB, the warp moves on at once). TMA clips at the tensor's edges only, so a short
      // row range that ends inside the output (a group or segment boundary) takes the plain stores.
      const bool tma_out = (p.out_tma != 0) && own && base != nullptr &&
                           (rows_valid == 32 || (!grouped && !fused));
      // A partial tile goes to its owner's slab the same way. Slabs are BM x BN whatever the
      // tile's valid extent, so whole windows are pushed and nothing needs clipping.
      const bool tma_push = kReduce && !own && (p.stage_tma != 0);
      // pull flavour: the stamp of a tile stored by TMA follows the completion of its bulk stores
      const bool stamp_late = tma_push || (kPull && pull && tma_out && rows_valid > 0);
      const CUtensorMap* tm_o = (kPull && pull) ? &p.tm_part[parity] : &p.tm_out;
      const int push_row0 = tma_push
          ? static_cast<int>(stage_slot_offset(sched, st_elt, p.stage_parity_bytes, parity, p.rank, ti.tile_in_seg) /
                             (static_cast<int64_t>(BN) * st_elt)) + row_base
          : 0;
      int groups_sent = 0;
      // A tile that ends at a segment boundary inside the matrix (column-split ownership) must not
      // store past its last column: TMA clips at the tensor's edge only, so such a window (its
      // unused half holds stale staging bytes) leaves by plain, clipped stores.
      const bool cols_by_tensor_edge = (ti.n0 + ti.cols >= sched.N);

      for (int win = 0; win < nwin; ++win) {
        if (win * groups_per_win * 32 >= ti.cols) break;
        const bool win_full = cols_by_tensor_edge || ((win + 1) * groups_per_win * 32 <= ti.cols);
        const bool win_tma_out = tma_out && win_full;
        // the store that read this staging buffer two windows ago must be done with it
        const uint32_t stg = stg_base + (win_count & 1u) * kEpiWinBytes;
        ++win_count;
        if (any_tma) {
          if (lane == 0) {
            // if the previous window left by TMA its store may still be reading the OTHER buffer;
            // a window sent by plain stores adds no group, so everything older has to be drained
            if (prev_win_tma) ptx::bulk_wait_group_read<1>();
            else ptx::bulk_wait_group_read<0>();
          }
          __syncwarp();
        }
        prev_win_tma = tma_push || (win_tma_out && rows_valid > 0);
        for (int h = 0; h < groups_per_win; ++h) {
          const int g = win * groups_per_win + h;
          const int col0 = g * 32;
          if (col0 >= ti.cols) break;
          uint32_t v[32];
          tick.lap(c_pub);
          if (CATCOC_BOUND_ABS(p, SITE_TMEM, acc * acc_stride + col0 + 32, KIND == KIND_MX ? 256 : kTmemCols)) {
            ptx::tmem_ld_32x32b_x32(taddr + static_cast<uint32_t>(col0), v);
            ptx::tcgen05_wait_ld();
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0u;
          }
          tick.lap(c_tld);
          if (g == last_group) {
            // every TMEM read of this tile is done: hand the accumulator back to the MMA warp
            ptx::tcgen05_fence_before();
            __syncwarp();
            if (lane == 0) {
              if (CTA2) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tail->acc_empty[acc]), 0u));
              else ptx::mbar_arrive(&tail->acc_empty[acc]);
            }
            released = true;
          }

          if (kScale && is_int && p.bias != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              const int c = ti.n0 + col0 + j;
              const int32_t b = (c < sched.N) ? __ldg(p.bias + nvec_off + c) : 0;
              v[j] = static_cast<uint32_t>(static_cast<int32_t>(v[j]) + b);
            }
          }

          if (kReduce && reduce_here && row_in_tile < ti.rows &&
              CATCOC_BOUND(p, SITE_FOLD_SLAB,
                           static_cast<int64_t>(parity) * p.stage_parity_bytes +
                               (static_cast<int64_t>(p.W - 1) * sched.tiles_per_seg + ti.tile_in_seg) * stage_tile_bytes(sched, pelt) +
                               (static_cast<int64_t>(row_in_tile) * BN + col0 + 32) * pelt,
                           LIM_STAGE)) {
            // fold the peers' partials in a fixed source order => deterministic sum. The loads of
            // two sources are issued back to back before their adds to keep more bytes in flight.
            const uint8_t* sbase = p.stage[p.rank] + (static_cast<int64_t>(row_in_tile) * BN + col0) * pelt;
            const int64_t slot_bytes = stage_tile_bytes(sched, pelt);
            const int64_t src_stride = static_cast<int64_t>(sched.tiles_per_seg) * slot_bytes;
            const int64_t base_off = static_cast<int64_t>(parity) * p.stage_parity_bytes + ti.tile_in_seg * slot_bytes;
            if (pelt == 2) {
              for (int s0 = 0; s0 < p.W; s0 += 2) {
                uint4 w[2][4];
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int src = s0 + j;
                  if (src < p.W && src != p.rank) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) w[j][u] = ptx::ld_global_v4(sbase + base_off + src * src_stride + u * 16);
                  }
                }
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                  const int src = s0 + j;
                  if (src < p.W && src != p.rank) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                      const uint32_t ww[4] = {w[j][u].x, w[j][u].y, w[j][u].z, w[j][u].w};
#pragma unroll
                      for (int e = 0; e < 4; ++e) {
                        const float2 f = unpack2(ww[e], pfmt);
                        v[u * 8 + e * 2] = __float_as_uint(__uint_as_float(v[u * 8 + e * 2]) + f.x);
                        v[u * 8 + e * 2 + 1] = __float_as_uint(__uint_as_float(v[u * 8 + e * 2 + 1]) + f.y);
                      }
                    }
                  }
                }
              }
            } else {
              for (int src = 0; src < p.W; ++src) {
                if (src == p.rank) continue;
                const uint8_t* sp = sbase + base_off + src * src_stride;
                uint4 w[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) w[u] = ptx::ld_global_v4(sp + u * 16);
#pragma unroll
                for (int u = 0; u < 8; ++u) {
                  const uint32_t ww[4] = {w[u].x, w[u].y, w[u].z, w[u].w};
#pragma unroll
                  for (int e = 0; e < 4; ++e) {
                    if (pfmt == FMT_S32)
                      v[u * 4 + e] = static_cast<uint32_t>(static_cast<int32_t>(v[u * 4 + e]) + static_cast<int32_t>(ww[e]));
                    else
                      v[u * 4 + e] = __float_as_uint(__uint_as_float(v[u * 4 + e]) + __uint_as_float(ww[e]));
                  }
                }
              }
            }
          }

          // convert this row's 32 values to the stored format and stage them
          if (st_fmt == FMT_S32 || (st_fmt == FMT_F32 && !is_int && !(dequant && own) && !affine && !(kScale && p.act != ACT_NONE))) {
#pragma unroll
            for (int u = 0; u < 8; ++u)
              stage_write(stg, lane, u,
                          make_uint4(v[u * 4], v[u * 4 + 1], v[u * 4 + 2], v[u * 4 + 3]));
          } else {
            float f[32];
            if (is_int) {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = static_cast<float>(static_cast<int32_t>(v[j]));
            } else {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            }
            if (kScale && dequant && own) {
              const int grow = ti.m0 + row_in_tile;
              const float sm =
                  (p.scale_m != nullptr && grow < sched.M) ? __ldg(p.scale_m + grow) : 1.0f;
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                const int c = ti.n0 + col0 + j;
                const float sn =
                    (p.scale_n != nullptr && c < sched.N) ? __ldg(p.scale_n + nvec_off + c) : 1.0f;
                f[j] = f[j] * sn * sm;
              }
            }
            if (kScale && affine) {
              // out = alpha * acc + beta * C + bias: each lane walks its own row of C
              const float alpha = p.alpha, beta = p.beta;
              const int cvalid = min(32, ti.cols - col0);
#pragma unroll
              for (int j = 0; j < 32; ++j) {
                float x = alpha * f[j];
                if (p.bias_f != nullptr && j < cvalid) x += __ldg(p.bias_f + nvec_off + ti.n0 + col0 + j);
                f[j] = x;
              }
              if (p.c_src != nullptr && row_in_tile < ti.rows) {
                const uint8_t* crow = static_cast<const uint8_t*>(p.c_src) +
                    (static_cast<int64_t>(ti.m0 + row_in_tile - p.out_row_shift) * p.ldc_src + ti.n0 + col0) * st_elt;
                if (cvalid == 32 && (reinterpret_cast<uintptr_t>(crow) & 15) == 0) {
                  if (st_fmt == FMT_F32) {
#pragma unroll
                    for (int u = 0; u < 8; ++u) {
                      const uint4 w = ptx::ld_global_v4(crow + u * 16);
                      f[u * 4] += beta * __uint_as_float(w.x);
                      f[u * 4 + 1] += beta * __uint_as_float(w.y);
                      f[u * 4 + 2] += beta * __uint_as_float(w.z);
                      f[u * 4 + 3] += beta * __uint_as_float(w.w);
                    }
                  } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                      const uint4 w = ptx::ld_global_v4(crow + u * 16);
                      const uint32_t ww[4] = {w.x, w.y, w.z, w.w};
#pragma unroll
                      for (int e = 0; e < 4; ++e) {
                        const float2 c2 = unpack2(ww[e], st_fmt);
                        f[u * 8 + e * 2] += beta * c2.x;
                        f[u * 8 + e * 2 + 1] += beta * c2.y;
                      }
                    }
                  }
                } else {
                  // ragged or unaligned: element loads (the index stays a compile-time constant
                  // so that f[] remains in registers)
#pragma unroll
                  for (int j = 0; j < 32; ++j) {
                    if (j < cvalid) {
                      float cv;
                      if (st_fmt == FMT_F32) {
                        cv = *reinterpret_cast<const float*>(crow + j * 4);
                      } else {
                        const uint32_t h = *reinterpret_cast<const uint16_t*>(crow + j * 2);
                        cv = unpack2(h, st_fmt).x;
                      }
                      f[j] += beta * cv;
                    }
                  }
                }
              }
            }
            if (kScale && p.act != ACT_NONE) {
#pragma unroll
              for (int j = 0; j < 32; ++j) f[j] = activate(f[j], p.act);
            }
            if (st_fmt == FMT_F32) {
#pragma unroll
              for (int u = 0; u < 8; ++u)
                stage_write(stg, lane, u,
                            make_uint4(__float_as_uint(f[u * 4]), __float_as_uint(f[u * 4 + 1]),
                                       __float_as_uint(f[u * 4 + 2]),
                                       __float_as_uint(f[u * 4 + 3])));
            } else {
#pragma unroll
              for (int u = 0; u < 4; ++u)
                stage_write(stg, lane, h * 4 + u,
                            make_uint4(pack2(f[u * 8], f[u * 8 + 1], st_fmt),
                                       pack2(f[u * 8 + 2], f[u * 8 + 3], st_fmt),
                                       pack2(f[u * 8 + 4], f[u * 8 + 5], st_fmt),
                                       pack2(f[u * 8 + 6], f[u * 8 + 7], st_fmt)));
            }
          }
        }
        __syncwarp();
        tick.lap(c_cvt);
        {
          const int per_win = 128 / st_elt;
          const int cols_valid = min(per_win, ti.cols - win * per_win);
          const int64_t wb = static_cast<int64_t>(win) * 128;
          if (!dst_ok) {
            // checked build: the destination lies outside its buffer; reported, nothing is stored
          } else if (tma_push) {
            ptx::fence_proxy_async_smem();
            __syncwarp();
            if (lane == 0) {
              ptx::tma_store_2d(&p.tm_stage[ti.seg], stg, win * per_win, push_row0);
              ptx::bulk_commit_group();
            }
            ++groups_sent;
          } else if (win_tma_out) {
            if (rows_valid > 0) {
              ptx::fence_proxy_async_smem();   // the staged bytes become visible to the TMA unit
              __syncwarp();
              if (lane == 0) {
                ptx::tma_store_2d(tm_o, stg, ti.n0 + win * per_win,
                                  static_cast<int>(ti.m0 + row_base - row_shift));
                ptx::bulk_commit_group();
              }
            }
          } else {
            flush_staged(stg, lane, base != nullptr ? base + wb : nullptr, pitch, rows_valid,
                         cols_valid, st_elt, vec_ok, mc != nullptr ? mc + wb : nullptr, peer_bases,
                         off + wb, p.rank, p.W);
          }
        }
        __syncwarp();
        tick.lap(c_flush);
      }
      if (reduce_here) tick.lap(c_own);
      if (!released) {
        // degenerate (empty) tile: nothing was read, still return the accumulator
        ptx::tcgen05_fence_before();
        __syncwarp();
        if (lane == 0) {
          if (CTA2) ptx::mbar_arrive_cluster(ptx::map_to_cta(ptx::smem_u32(&tail->acc_empty[acc]), 0u));
          else ptx::mbar_arrive(&tail->acc_empty[acc]);
        }
      }

      // ---- publish this warp's quarter of the tile ----
      if (kPull && pull) {
        // Tell the tile's owner that this rank's partial rows are in place. Plain stores are ordered
        // before the release by the warp barrier; TMA stores must have completed first. They go to
        // local memory, so the wait is short, and the accumulator was handed back before it: unlike
        // a push over the link this costs less than announcing the tile one tile late would (with a
        // deep K the next tile ends tens of microseconds later, and the owner would sit idle).
        __syncwarp();
        if (lane == 0 && !p.withhold_signals) {
          if (stamp_late) {
            ptx::bulk_wait_group_all();
            ptx::fence_proxy_async();
          }
          const int64_t si = arrive_flag_index(sched, ti.tile_in_seg, p.rank) * qpt + qid;
          if (CATCOC_BOUND(p, SITE_ARRIVE_POST, si + 1, LIM_ARRIVE)) ptx::st_release_sys_u32(p.arrive[ti.seg] + si, epoch);
        }
      } else if (kReduce && fused && (p.mode == MODE_RS || p.mode == MODE_AR) && (!own || p.mode == MODE_AR)) {
        // Data stores of all 32 lanes happen-before lane 0's release through the warp barrier;
        // the release is cumulative, so one system-scope release by one lane publishes them all.
        __syncwarp();
        tick.lap(c_work);
        if (!p.withhold_signals) {
          if (!own) {
            const int64_t si = arrive_flag_index(sched, ti.tile_in_seg, p.rank) * qpt + qid;
            uint32_t* stamp = p.arrive[ti.seg] + si;
            if (!CATCOC_BOUND(p, SITE_ARRIVE_POST, si + 1, LIM_ARRIVE)) {
              // checked build: reported, no stamp
            } else if (tma_push) {
              // the stores of the tile before this one are complete once at most this tile's
              // groups are in flight: announce that tile now, this one a tile later
              if (lane == 0 && pending_stamp != nullptr) {
                // (the count is an immediate: take the largest one not above this tile's groups)
                if (groups_sent >= 8) ptx::bulk_wait_group<8>();
                else if (groups_sent >= 4) ptx::bulk_wait_group<4>();
                else if (groups_sent >= 2) ptx::bulk_wait_group<2>();
                else if (groups_sent == 1) ptx::bulk_wait_group<1>();
                else ptx::bulk_wait_group_all();
                ptx::fence_proxy_async();
                ptx::st_release_sys_u32(pending_stamp, epoch);
              }
              pending_stamp = stamp;
            } else if (lane == 0) {
              ptx::st_release_sys_u32(stamp, epoch);
            }
          } else {
            // the reduced rows are in every rank's output: stamp them everywhere
            const int gid = (ti.seg * sched.tiles_per_seg + ti.tile_in_seg) * qpt + qid;
            if (!CATCOC_BOUND(p, SITE_DONE_POST, gid + 1, LIM_DONE)) {
              // checked build: reported, no stamp
            } else if (p.done_mc != nullptr && mc != nullptr) {
              if (lane == 0) ptx::multimem_st_release_u32(p.done_mc + gid, epoch);
            } else if (lane < p.W) {
              ptx::st_release_sys_u32(p.done[lane] + gid, epoch);
            }
          }
        }
      }

      tick.lap(c_pub);
      if (lane == 0 && q == 0) emit_event(p, EV_EPILOGUE, EV_END, static_cast<uint32_t>(t));
      if (tr) {
        const unsigned long long dt = static_cast<unsigned long long>(ptx::clock_cycles() - tile_t0);
        if (own) c_tile_own += dt; else c_tile_push += dt;
      }
      acc ^= 1;
      if (acc == 0) acc_phase ^= 1u;
    }

    // every TMA store of this warp has to be performed before the kernel ends, and the last
    // pushed tile is still unannounced
    if (kReduce || kPull) settle_pending();
    if (any_tma && lane == 0) ptx::bulk_wait_group_all();
    __syncwarp();
    tick.lap(c_work);
    if (tr) {
      atomicAdd(p.trace + 5, c_full); atomicAdd(p.trace + 6, c_work); atomicAdd(p.trace + 7, c_peer);
      atomicAdd(p.trace + 9, c_pub); atomicAdd(p.trace + 10, c_own);
      atomicAdd(p.trace + 11, c_tld); atomicAdd(p.trace + 12, c_cvt); atomicAdd(p.trace + 13, c_flush);
      atomicAdd(p.trace + 14, c_tile_own); atomicAdd(p.trace + 15, c_tile_push);
    }

    // all-reduce tail: this rank's output is complete only when every owner's tiles landed
    if ((kReduce || kPull) && fused && p.mode == MODE_AR && ok && !*abort_flag) {
      const int et = (warp - 2) * 32 + lane;
      const int nstamps = sched.total_tiles * qpt * ((kPull && pull) ? kPullStrips : 1);
      for (int j = blockIdx.x + et * gridDim.x; j < nstamps; j += gridDim.x * kEpiWarps * 32) {
        uint32_t seen = 0;
        if (!CATCOC_BOUND(p, SITE_DONE_POLL, j + 1, LIM_DONE)) break;
        if (!wait_stamp(p.done[p.rank] + j, epoch, p.timeout_ns, abort_flag, &seen)) {
          report_status(p, STATUS_TIMEOUT_DONE, static_cast<uint32_t>(j), epoch, seen,
                        static_cast<uint32_t>((j / qpt) / sched.tiles_per_seg));
          *abort_flag = 1;
          break;
        }
      }
    }
  } else if (warp == 2 + kEpiWarps) {
    // =============================== TMA producer for B ===============================
    // Operand loading is split over two warps (this one and warp 0) because one warp cannot
    // issue both operands' copies fast enough to keep the tensor core fed.
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    GroupWalk walk = group_walk_begin(p);
    for (int t = worker; ok && t < total_tiles; t += num_workers) {
      const TileInfo ti = walk_tile(p, t, walk);
      int b_col = ti.n0 + sub * b_cols_cta;
      int b_k_off = 0;
      if (grouped) {
        b_col += ti.seg * p.g_b_row;
        b_k_off = ti.seg * p.g_b_k;
      }
      for (int kb = 0; kb < num_kb; ++kb) {
        if (!ptx::mbar_wait(&tail->empty[stage], phase ^ 1u, p.timeout_ns, abort_flag)) {
          if (lane == 0) {
            report_status(p, STATUS_TIMEOUT_PIPELINE, 4u, static_cast<uint32_t>(t), static_cast<uint32_t>(kb), 0u);
            *abort_flag = 1;
          }
          ok = false;
          break;
        }
        if (ptx::elect_one()) {
          const int per_box = 128 / p.elt_bytes_a;
          const uint32_t bar = CTA2 ? ptx::map_to_cta(ptx::smem_u32(&tail->full[stage]), 0u) : 0u;
          if (KIND == KIND_MX) {
            const int nblk = BN / 128;
            ptx::mbar_expect_tx(&tail->full[stage], b_stage_bytes + nblk * 512);
            for (int j = 0; j < nblk; ++j)
              ptx::bulk_load_1d(smem + stage * kStageBytes + kSfSmemOff + 512 * (1 + j),
                                p.sfb + (static_cast<int64_t>(b_col / 128 + j) * p.sf_k_blocks + kb) * 512, 512,
                                &tail->full[stage]);
          } else if (!CTA2) ptx::mbar_expect_tx(&tail->full[stage], kps * b_stage_bytes);
          else if (leader) ptx::mbar_expect_tx(&tail->full[stage], 2u * kps * b_stage_bytes);
#pragma unroll
          for (int j = 0; j < 2; ++j) {
            if (j >= kps) break;
            uint8_t* sb = smem + stage * kStageBytes + j * sub_bytes + kABytes;
            const int k0 = (kb * kps + j) * p.bk + b_k_off;
            if (!CTA2) {
              if (!p.b_mn_major) {
                ptx::tma_load_2d(sb, &p.tm_b, &tail->full[stage], k0, b_col);
              } else if (p.b_3d) {
                ptx::tma_load_3d(sb, &p.tm_b, &tail->full[stage], 0, k0, b_col / per_box);
              } else {
                for (int b = 0; b < b_cols_cta / per_box; ++b)
                  ptx::tma_load_2d(sb + b * (p.bk * 128), &p.tm_b, &tail->full[stage], b_col + b * per_box, k0);
              }
            } else {
              if (!p.b_mn_major) {
                ptx::tma_load_2d_pair(sb, &p.tm_b, bar, k0, b_col);
              } else if (p.b_3d) {
                ptx::tma_load_3d_pair(sb, &p.tm_b, bar, 0, k0, b_col / per_box);
              } else {
                for (int b = 0; b < b_cols_cta / per_box; ++b)
                  ptx::tma_load_2d_pair(sb + b * (p.bk * 128), &p.tm_b, bar, b_col + b * per_box, k0);
              }
            }
          }
        }
        __syncwarp();
        if (++stage == kStages) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    // ======================= communication warps =======================
    const int cw = warp - (3 + kEpiWarps);               // this communication warp ...
    const int ncw = static_cast<int>(blockDim.x >> 5) - (3 + kEpiWarps);   // ... of so many per CTA
    if (fused && p.mode == MODE_AG) {
      // All-gather: send this rank's A shard into every rank's gathered buffer in units of
      // chunk_rows x 512 B. With the multicast alias one multimem.st per 16 bytes reaches every
      // rank (the shard leaves this GPU once), chunk-major: the consumers visit the chunks of all
      // peers side by side. Without it the units go to one peer after the other, the peer that
      // consumes the shard first is served first.
      const GatherPlan& gp = p.gp;
      const bool mcast = (p.gathered_mc != nullptr) && (p.gflags_mc != nullptr);
      const int units_per_peer = gp.n_chunks * gp.n_slices;
      const int64_t total_units = mcast ? units_per_peer : static_cast<int64_t>(p.W) * units_per_peer;
      const int slice_bytes = gp.slice_cols * p.elt_bytes_a;   // <= 512
      const int64_t row_bytes = static_cast<int64_t>(gp.K) * p.elt_bytes_a;
      if (lane == 0) emit_event(p, EV_COMM, EV_BEGIN, static_cast<uint32_t>(cw));
      for (int64_t u = static_cast<int64_t>(blockIdx.x) * ncw + cw; u < total_units;
           u += static_cast<int64_t>(gridDim.x) * ncw) {
        if (*abort_flag) break;
        const int step = static_cast<int>(u / units_per_peer);  // W-1 remote peers, then local
        const int rem = static_cast<int>(u - static_cast<int64_t>(step) * units_per_peer);
        const int chunk = rem / gp.n_slices;
        const int slice = rem - chunk * gp.n_slices;
        const int peer = (step == p.W - 1) ? p.rank : peer_for_push_ag(p.rank, step + 1, p.W);
        const int r0 = chunk * gp.chunk_rows;
        const int nrows = min(gp.chunk_rows, gp.m - r0);
        const int64_t cb = static_cast<int64_t>(slice) * slice_bytes + lane * 16;
        // bytes of this lane's 16-byte unit that hold shard data (a raw shard may end inside the unit; the
        // rest of a gathered row is padding that nobody reads, zero-filled here)
        const int64_t src_row_bytes = p.ag_raw ? p.a_row_bytes : row_bytes;
        const int valid = static_cast<int>(min(static_cast<int64_t>(16), src_row_bytes - cb));
        const bool col_ok = (lane * 16 < slice_bytes) && (cb + 16 <= row_bytes);
        const bool plain = (p.ag_raw == 0) || (p.a_vec == 16 && valid == 16);
        const uint8_t* src = p.a_local + static_cast<int64_t>(r0) * p.a_local_pitch + cb;
        uint8_t* dstp = (mcast ? p.gathered_mc : p.gathered[peer]) +
                        static_cast<int64_t>(parity) * p.gathered_parity_bytes +
                        (static_cast<int64_t>(p.rank) * gp.m + r0) * p.gathered_pitch + cb;
        [[maybe_unused]] const int64_t dst_end = static_cast<int64_t>(parity) * p.gathered_parity_bytes +
                                                 (static_cast<int64_t>(p.rank) * gp.m + r0 + nrows - 1) * p.gathered_pitch + cb + 16;
        if (col_ok && nrows > 0 && CATCOC_BOUND(p, SITE_GATHER_PUSH, dst_end, LIM_GATHERED)) {
          // 16 rows (8 KiB per warp) in flight per round trip: the copy is latency bound, which is
          // why several warps per CTA share it
          for (int r = 0; r < nrows; r += 16) {
            uint4 buf[16];
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (r + i < nrows) {
                const uint8_t* sp = src + static_cast<int64_t>(r + i) * p.a_local_pitch;
                buf[i] = plain ? ptx::ld_global_nc_v4(sp) : load16_pieces(sp, p.a_vec, valid);
              }
            if (mcast) {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (r + i < nrows)
                  ptx::multimem_st_v4(dstp + static_cast<int64_t>(r + i) * p.gathered_pitch, buf[i]);
            } else {
#pragma unroll
              for (int i = 0; i < 16; ++i)
                if (r + i < nrows)
                  ptx::st_global_v4(dstp + static_cast<int64_t>(r + i) * p.gathered_pitch, buf[i]);
            }
          }
        }
        // all lanes' stores happen-before lane 0's release through the warp barrier (cumulative)
        __syncwarp();
        if (lane == 0 && !p.withhold_signals) {
          const int64_t fi = gather_flag_index(gp, p.rank, chunk, slice);
          if (!CATCOC_BOUND(p, SITE_GFLAG_POST, fi + 1, LIM_GFLAGS)) {
            // checked build: reported, no stamp
          } else if (mcast) ptx::multimem_st_release_u32(p.gflags_mc + fi, epoch);
          else ptx::st_release_sys_u32(p.gflags[peer] + fi, epoch);
        }
      }
      if (lane == 0) emit_event(p, EV_COMM, EV_END, static_cast<uint32_t>(cw));
    } else if (kPull && pull) {
      // Reducer warps of the pull flavour. Task j = (i-th tile of MY segment in visiting order, a
      // 32-row quarter of it, an 8-row strip of the quarter), dealt out round-robin over all reducer
      // warps of the grid so that the tiles that finish first are reduced first. A strip is one
      // batch of loads per lane: after the last tile of the launch the whole grid's reducer warps
      // share what is left, each with a single round trip through the switch. A task waits until every rank's stamp for
      // that quarter is in, reads the sum of the W partial copies through the switch
      // (multimem.ld_reduce, fp32 accumulation) and stores it: into `out` (reduce-scatter) or, with
      // one multimem.st per 16 bytes, into every rank's output followed by a `done` stamp
      // (all-reduce). Nothing in the GEMM pipeline ever waits for these warps.
      const int gw = static_cast<int>(blockIdx.x) * ncw + cw;
      const int total_gw = static_cast<int>(gridDim.x) * ncw;
      const int tasks = sched.tiles_per_seg * qpt * kPullStrips;
      const bool bf = (p.partial_fmt == FMT_BF16);
      const uint8_t* src_base = p.part_mc + static_cast<int64_t>(parity) * p.part_parity_bytes;
      const bool ar = (p.mode == MODE_AR);
      uint8_t* dst_base = ar ? p.ar_out_mc + static_cast<int64_t>(parity) * p.ar_out_parity_bytes
                             : static_cast<uint8_t*>(p.out);
      bool ok = true;
      for (int j = gw; ok && j < tasks; j += total_gw) {
        if (*abort_flag) break;
        const int strip = j % kPullStrips;
        const int jq = j / kPullStrips;
        const int i = jq / qpt, qd = jq - i * qpt;
        const TileInfo ti = seg_tile(sched, p.rank, i);
        const int row0 = qd * 32 + strip * (32 / kPullStrips);
        const int rows_valid = max(0, min(32 / kPullStrips, ti.rows - row0));
        if (rows_valid > 0 && ti.cols > 0) {
          for (int src = lane; src < p.W; src += 32) {
            uint32_t seen = 0;
            const int64_t idx = arrive_flag_index(sched, ti.tile_in_seg, src) * qpt + qd;
            if (!CATCOC_BOUND(p, SITE_ARRIVE_POLL, idx + 1, LIM_ARRIVE)) {
              ok = false;
            } else if (!wait_stamp(p.arrive[p.rank] + idx, epoch, p.timeout_ns, abort_flag, &seen, 200)) {
              report_status(p, STATUS_TIMEOUT_ARRIVE, static_cast<uint32_t>(ti.tile_in_seg), epoch, seen,
                            static_cast<uint32_t>(src));
              *abort_flag = 1;
              ok = false;
            }
          }
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          ptx::fence_acq_rel_sys();   // the other lanes' acquires order this lane's loads too
          if (lane == 0) emit_event(p, EV_REDUCER, EV_BEGIN, static_cast<uint32_t>(j));
          const int upr = (ti.cols * 2 + 15) >> 4;          // 16-byte units per row
          const int total_units = rows_valid * upr;
          const int64_t src_row0 = (static_cast<int64_t>(ti.m0 + row0) * p.ldp + ti.n0) * 2;
          const int64_t dst_row0 = (static_cast<int64_t>(ti.m0 + row0 - (ar ? 0 : p.out_row_shift)) * p.ldc + ti.n0) * 2;
          [[maybe_unused]] const int64_t row_span = static_cast<int64_t>(upr) * 16;
          const bool io_ok =
              CATCOC_BOUND(p, SITE_PART_REDUCE, static_cast<int64_t>(parity) * p.part_parity_bytes + src_row0 +
                                                    static_cast<int64_t>(rows_valid - 1) * p.ldp * 2 + row_span, LIM_PART) &&
              (ar ? CATCOC_BOUND(p, SITE_AR_OUT, static_cast<int64_t>(parity) * p.ar_out_parity_bytes + dst_row0 +
                                                     static_cast<int64_t>(rows_valid - 1) * p.ldc * 2 + row_span, LIM_AR_OUT)
                  : CATCOC_BOUND(p, SITE_OUT_STORE, dst_row0 + static_cast<int64_t>(rows_valid - 1) * p.ldc * 2 + row_span,
                                 LIM_OUT));
          for (int u0 = 0; io_ok && u0 < total_units; u0 += 32 * 8) {
            uint4 v[8];
            int64_t doff[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int u = u0 + k * 32 + lane;
              if (u < total_units) {
                const int r = u / upr, c = u - r * upr;
                const uint8_t* sp = src_base + src_row0 + static_cast<int64_t>(r) * p.ldp * 2 + c * 16;
                doff[k] = dst_row0 + static_cast<int64_t>(r) * p.ldc * 2 + c * 16;
                v[k] = bf ? ptx::multimem_ld_reduce_add_bf16x2_v4(sp) : ptx::multimem_ld_reduce_add_f16x2_v4(sp);
              }
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
              const int u = u0 + k * 32 + lane;
              if (u < total_units) {
                if (ar) ptx::multimem_st_v4(dst_base + doff[k], v[k]);
                else ptx::st_global_v4(dst_base + doff[k], v[k]);
              }
            }
          }
        }
        if (lane == 0 && rows_valid > 0) emit_event(p, EV_REDUCER, EV_END, static_cast<uint32_t>(j));
        if (ar) {
          // the reduced rows are in every rank's output: stamp them everywhere
          __syncwarp();
          if (lane == 0 && !p.withhold_signals) {
            const int gid = ((p.rank * sched.tiles_per_seg + ti.tile_in_seg) * qpt + qd) * kPullStrips + strip;
            if (CATCOC_BOUND(p, SITE_DONE_POST, gid + 1, LIM_DONE)) ptx::multimem_st_release_u32(p.done_mc + gid, epoch);
          }
        }
      }
    }
  }

  // =============================== teardown ===============================
  ptx::tcgen05_fence_before();
  __syncthreads();
  if (CTA2) ptx::cluster_sync_all();   // neither CTA of a pair leaves while the other may touch it
  ptx::tcgen05_fence_after();
  if (warp == 1) {
    if (CTA2) ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    else ptx::tmem_dealloc(tmem_base, kTmemCols);
  }
  if (p.trace != nullptr && threadIdx.x == 0)
    atomicAdd(p.trace + 8, static_cast<unsigned long long>(ptx::clock_cycles() - cta_t0));
  if (fused && threadIdx.x == 0) {
    // the last CTA to finish publishes the new epoch for the next launch on this stream
    __threadfence();
    const uint32_t prev = atomicAdd(p.cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.cta_counter = 0;
      if (!*abort_flag && *p.status == 0u) *p.epoch_ptr = epoch;
      __threadfence();
    }
  }
}

}  // namespace catcoc
