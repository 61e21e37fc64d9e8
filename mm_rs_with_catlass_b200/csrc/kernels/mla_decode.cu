// Multi-head latent attention, decode step over a paged latent cache, on tcgen05.
//
// Every query head shares ONE key / value stream: the 512-wide latent (keys and values at once) plus a 64-wide
// rotary part that only the scores see. A CTA owns up to 128 query rows (rows = new tokens x heads of one batch
// item), one half of the 512 output columns and one slice of the sequence:
//
//   warps 0..3  softmax      : one query row per thread: tcgen05.ld 32 scores, exp2, row sum, P written back over the
//                              scores (tcgen05.st), O rescaled in TMEM when the reference maximum moved
//   warp 4      TMA producer : the Q rows once, then 32 keys per step through a ring of slots (two copies per step:
//                              the eight latent blocks at once, the rotary block); the page of every step comes from
//                              the block table
//   warp 5      MMA issuer   : S = Q K^T (36 MMAs over the 576 columns) one step ahead of O += P V (P from TMEM,
//                              V = this CTA's 256 latent columns of the same slot, MN-major)
//
// TMEM: two score buffers of 32 columns, O in 256 columns. Shared memory holds Q (the largest item: 128 rows x
// 576 columns = 144 KiB, which leaves two 36 KiB slots; 64 rows when the batch item has no more, which leaves four)
// and the ring. The two CTAs that share a batch item and a slice sit side by side in the grid, so the second read
// of a key block comes from L2. With more than one slice per sequence the partial (O, m, l) go to a workspace and
// mla_combine_kernel merges them (flash decoding).
//
// The reference carries this computation as 3rdparty/catlass/examples/19_mla/mla_kernel.cpp (paged cache of 128-key
// pages, 1..4 new tokens per sequence, optional causal mask among the new tokens); inputs and golden follow its
// gen_data.py: q_nope [T, H, 512], q_rope [T, H, 64], latent cache [pages, 128, 512], rope cache [pages, 128, 64],
// block table [B, max_pages], scale = 1 / sqrt(576).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstring>
#include "catcoc/capi.h"
#include "catcoc/host_util.h"
#include "catcoc/params.h"
#include "catcoc/ptx.cuh"

namespace catcoc {
namespace mla {

constexpr int kDV = 512;            // latent width (values, and the first part of the keys)
constexpr int kDR = 64;             // rotary width (keys only)
constexpr int kChunks = (kDV + kDR) / 64;   // 64-column blocks of a key row: 8 latent + 1 rotary
constexpr int kPage = 128;          // keys per cache page
constexpr int kBKV = 32;            // keys per step
constexpr int kHalf = 256;          // output columns per CTA
constexpr int kThreads = 192;
constexpr int kProducerWarp = 4, kIssuerWarp = 5;
constexpr int kKChunkBytes = kBKV * 128;            // 32 keys x 64 columns
constexpr int kSlotBytes = kChunks * kKChunkBytes;  // 36 KiB
constexpr int kMaxSlots = 4;
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kOCol = 64;
constexpr float kLazyRescale = 8.0f;

struct MlaParams {
  // The 512 latent columns are described as {64, rows, 8 blocks} (the block stride is 128 bytes, smaller than the row
  // stride): ONE copy then fills all eight 64-column blocks of a tile, block-major, each 128-byte swizzled.
  CUtensorMap tm_qn, tm_qr;       // q_nope {64, rows, 8}, box {64, QR, 8} / q_rope {64, rows}, box {64, QR}
  CUtensorMap tm_kn, tm_kr;       // latent cache {64, 128, 8, pages}, box {64, 32, 8, 1} / rope cache {64, 128, pages}, box {64, 32, 1}
  const int* block_table;         // [B, max_pages]
  const int* kv_lens;             // [B]
  void* out;                      // [rows, 512] operand dtype
  float* part_o;                  // [splits, rows, 512] (splits > 1)
  float* part_ml;                 // [splits, rows, 2]
  int B, q_len, H, max_pages, num_pages, splits;
  int rows_per_item, chunks_per_item, total_rows;
  int causal;
  float scale_log2;
  int fmt;
  uint32_t idesc_qk, idesc_pv;
  uint32_t* status;
  uint64_t timeout_ns;
};

struct Bars {
  uint64_t q_full, kv_full[kMaxSlots], kv_empty[kMaxSlots], s_full[2], p_full[2], pv_done, o_final;
  uint32_t tmem_base, abort_flag;
};

CATCOC_DEVICE void fail(const MlaParams& p, uint32_t what, uint32_t a, uint32_t b) {
  if (atomicCAS(p.status, 0u, static_cast<uint32_t>(STATUS_TIMEOUT_PIPELINE)) == 0u) {
    p.status[1] = 0u; p.status[2] = 200u + what; p.status[3] = a; p.status[4] = b; p.status[5] = 0u;
    p.status[6] = blockIdx.y;
    __threadfence_system();
  }
}

CATCOC_DEVICE uint32_t pack16(float lo, float hi, int fmt) {
  if (fmt == FMT_BF16) { __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&hh); }
  __half2 hh = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&hh);
}

// QR: query rows held in shared memory (64 or 128). The MMA always spans 128 rows; with QR = 64 the upper 64 rows of
// every Q block alias the bytes that follow it (more of Q, then the ring): finite values whose scores land in TMEM
// lanes 64..127, which nobody stores.
template <int QR>
__global__ void __launch_bounds__(kThreads, 1) mla_decode_kernel(const __grid_constant__ MlaParams p) {
  constexpr int kQChunkBytes = QR * 128;
  constexpr int kQBytes = kChunks * kQChunkBytes;
  constexpr int kSlots = QR == 64 ? 4 : 2;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;
  uint8_t* skv = sq + kQBytes;
  Bars* bars = reinterpret_cast<Bars*>(skv + kSlots * kSlotBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int half = blockIdx.x;                                    // which 256 output columns
  const int item = blockIdx.y / p.chunks_per_item;                // batch item
  const int chunk = blockIdx.y - item * p.chunks_per_item;        // 128-row chunk of its tokens x heads
  const int split = blockIdx.z;
  const int row_in_item0 = chunk * 128;
  const int grow0 = item * p.rows_per_item + row_in_item0;        // first global row of this CTA
  const int kv_len = min(max(0, p.kv_lens[item]), p.max_pages * kPage);
  // steps of 32 keys this slice walks
  const int steps_total = (kv_len + kBKV - 1) / kBKV;
  const int steps_per_split = (steps_total + p.splits - 1) / p.splits;
  const int step0 = min(steps_total, split * steps_per_split);
  const int nsteps = min(steps_total, step0 + steps_per_split) - step0;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kSlots; ++s) { ptx::mbar_init(&bars->kv_full[s], 1); ptx::mbar_init(&bars->kv_empty[s], 1); }
    for (int i = 0; i < 2; ++i) { ptx::mbar_init(&bars->s_full[i], 1); ptx::mbar_init(&bars->p_full[i], 4); }
    ptx::mbar_init(&bars->pv_done, 1);
    ptx::mbar_init(&bars->o_final, 1);
    bars->abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&p.tm_qn); ptx::prefetch_tmap(&p.tm_qr); ptx::prefetch_tmap(&p.tm_kn); ptx::prefetch_tmap(&p.tm_kr);
  }
  if (warp == kIssuerWarp) { ptx::tmem_alloc(&bars->tmem_base, kTmemCols); ptx::tmem_relinquish(); }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (nsteps > 0 && ptx::elect_one()) {
      ptx::mbar_expect_tx(&bars->q_full, kQBytes);
      ptx::tma_load_3d(sq, &p.tm_qn, &bars->q_full, 0, grow0, 0);
      ptx::tma_load_2d(sq + (kChunks - 1) * kQChunkBytes, &p.tm_qr, &bars->q_full, 0, grow0);
    }
    __syncwarp();
    int cached_pi = -1, cached_page = 0;
    for (int i = 0; i < nsteps; ++i) {
      const int slot = i % kSlots;
      const uint32_t use = static_cast<uint32_t>(i / kSlots);
      const int key0 = (step0 + i) * kBKV;
      if (key0 / kPage != cached_pi) {               // every lane reads the entry: its latency hides behind the wait below
        cached_pi = key0 / kPage;
        cached_page = __ldg(p.block_table + static_cast<int64_t>(item) * p.max_pages + cached_pi);
        cached_page = min(max(cached_page, 0), p.num_pages - 1);   // a bad entry reads a wrong page, never outside the cache
      }
      if (!ptx::mbar_wait(&bars->kv_empty[slot], (use & 1u) ^ 1u, p.timeout_ns, abort_flag)) {
        if (lane == 0) { fail(p, 1u, i, 0u); *abort_flag = 1; }
        break;
      }
      if (ptx::elect_one()) {
        const int page = cached_page;
        const int prow = key0 % kPage;
        uint8_t* dst = skv + slot * kSlotBytes;
        ptx::mbar_expect_tx(&bars->kv_full[slot], kSlotBytes);
        ptx::tma_load_4d(dst, &p.tm_kn, &bars->kv_full[slot], 0, prow, 0, page);
        ptx::tma_load_3d(dst + (kChunks - 1) * kKChunkBytes, &p.tm_kr, &bars->kv_full[slot], 0, prow, page);
      }
      __syncwarp();
    }
  } else if (warp == kIssuerWarp) {
    // ------------------------------ MMA issuer ------------------------------
    auto wait_kv = [&](int i) {
      return ptx::mbar_wait(&bars->kv_full[i % kSlots], static_cast<uint32_t>(i / kSlots) & 1u, p.timeout_ns, abort_flag);
    };
    auto issue_qk = [&](int i) {
      // S[128, 32 keys] = Q[128, 576] K^T: both K-major, 64-column blocks, 16 columns per MMA
      const uint32_t kbase = ptx::smem_u32(skv + (i % kSlots) * kSlotBytes);
#pragma unroll
      for (int c = 0; c < kChunks; ++c) {
        const uint64_t dq = ptx::make_smem_desc_sw128(ptx::smem_u32(sq + c * kQChunkBytes), 16u, 1024u);
        const uint64_t dk = ptx::make_smem_desc_sw128(kbase + c * kKChunkBytes, 16u, 1024u);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          ptx::umma_f16(tmem + (i & 1) * kBKV, dq + static_cast<uint64_t>(kk * 2), dk + static_cast<uint64_t>(kk * 2), p.idesc_qk,
                        (c | kk) != 0 ? 1u : 0u);
      }
      ptx::tcgen05_commit(&bars->s_full[i & 1]);
    };
    auto issue_pv = [&](int i) {
      // O[128, 256] += P[128, 32 keys] V[32 keys, 256]: P from TMEM (8 columns per 16 keys), V = blocks 4 half .. 4 half + 3
      // of the slot, MN-major: 16 key rows per MMA = 2048 bytes down a block, blocks one K chunk apart
      const uint64_t dv = ptx::make_smem_desc_sw128(ptx::smem_u32(skv + (i % kSlots) * kSlotBytes + half * 4 * kKChunkBytes),
                                                    static_cast<uint32_t>(kKChunkBytes), 1024u);
#pragma unroll
      for (int kk = 0; kk < kBKV / 16; ++kk)
        ptx::umma_f16_ts(tmem + kOCol, tmem + (i & 1) * kBKV + kk * 8, dv + static_cast<uint64_t>((kk * 2048) >> 4), p.idesc_pv,
                         (i > 0 || kk != 0) ? 1u : 0u);
      ptx::tcgen05_commit(&bars->kv_empty[i % kSlots]);
      // pv_done is waited on only by a softmax step that rescales O, so its phases are not all consumed: the end of
      // the walk gets a barrier of its own, whose single phase cannot be mistaken for an earlier one
      if (i + 1 < nsteps) ptx::tcgen05_commit(&bars->pv_done);
      else ptx::tcgen05_commit(&bars->o_final);
    };
    bool ok = true;
    if (nsteps > 0) {
      ok = ptx::mbar_wait(&bars->q_full, 0u, p.timeout_ns, abort_flag) && wait_kv(0);
      if (ok) {
        ptx::tcgen05_fence_after();
        if (ptx::elect_one()) issue_qk(0);
        __syncwarp();
      }
    }
    for (int i = 0; ok && i < nsteps; ++i) {
      if (i + 1 < nsteps) {
        // the scores of the next step go to the other buffer while the softmax warps work on this one
        ok = wait_kv(i + 1);
        if (!ok) break;
        ptx::tcgen05_fence_after();
        if (ptx::elect_one()) issue_qk(i + 1);
        __syncwarp();
      }
      ok = ptx::mbar_wait(&bars->p_full[i & 1], static_cast<uint32_t>(i >> 1) & 1u, p.timeout_ns, abort_flag);
      if (!ok) break;
      ptx::tcgen05_fence_after();
      if (ptx::elect_one()) issue_pv(i);
      __syncwarp();
    }
    if (!ok && lane == 0) { fail(p, 2u, 0u, 0u); *abort_flag = 1; }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int row = warp * 32 + lane;                // query row inside the chunk == TMEM lane
    const int row_in_item = row_in_item0 + row;
    const bool row_valid = row_in_item < p.rows_per_item;
    const int tok = min(row_in_item / p.H, p.q_len - 1);
    // keys [0, vis) are visible: with the causal mask new token t does not see the new tokens behind it
    const int vis = p.causal ? max(0, kv_len - (p.q_len - 1 - tok)) : kv_len;
    const int vis_all = p.causal ? max(0, kv_len - (p.q_len - 1)) : kv_len;
    const uint32_t lane_base = tmem + (static_cast<uint32_t>(warp * 32) << 16);
    const uint32_t t_o = lane_base + kOCol;
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int i = 0; i < nsteps; ++i) {
      if (!ptx::mbar_wait(&bars->s_full[i & 1], static_cast<uint32_t>(i >> 1) & 1u, p.timeout_ns, abort_flag)) { ok = false; break; }
      ptx::tcgen05_fence_after();
      const uint32_t t_s = lane_base + (i & 1) * kBKV;
      const int key0 = (step0 + i) * kBKV;
      const bool masked = key0 + kBKV > vis_all;
      uint32_t v[32];
      ptx::tmem_ld_32x32b_x32(t_s, v);
      ptx::tcgen05_wait_ld();
      float mx = -INFINITY;
#pragma unroll
      for (int k = 0; k < 32; ++k)
        if (!masked || key0 + k < vis) mx = fmaxf(mx, __uint_as_float(v[k]));
      const float m_new = fmaxf(m_ref, mx * sc);
      const bool move = __any_sync(0xffffffffu, m_new > m_ref + kLazyRescale);
      const float m_use = move ? m_new : m_ref;
      const float m_safe = (m_use == -INFINITY) ? 0.0f : m_use;
      const float alpha = !move ? 1.0f : ((m_ref == -INFINITY) ? 0.0f : ptx::ex2_approx(m_ref - m_safe));
      float sum = 0.0f;
      uint32_t w[16];
#pragma unroll
      for (int k = 0; k < 32; k += 2) {
        float e0 = ptx::ex2_approx(fmaf(__uint_as_float(v[k]), sc, -m_safe));
        float e1 = ptx::ex2_approx(fmaf(__uint_as_float(v[k + 1]), sc, -m_safe));
        if (masked) {
          if (key0 + k >= vis) e0 = 0.0f;
          if (key0 + k + 1 >= vis) e1 = 0.0f;
        }
        sum += e0 + e1;
        w[k >> 1] = pack16(e0, e1, p.fmt);
      }
      ptx::tmem_st_32x32b_x16(t_s, w);
      l = l * alpha + sum;
      m_ref = m_use;
      if (move && i > 0) {
        // O must hold every product issued so far before it is rescaled. P V of step i - 2 completed before the scores of
        // this step did (issue order), P V of step i cannot start before this warp arrives below: the barrier is in
        // phase i - 1 or i, never further, so the parity is unambiguous.
        if (!ptx::mbar_wait(&bars->pv_done, static_cast<uint32_t>(i - 1) & 1u, p.timeout_ns, abort_flag)) { ok = false; break; }
        ptx::tcgen05_fence_after();
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t o[32];
          ptx::tmem_ld_32x32b_x32(t_o + c * 32, o);
          ptx::tcgen05_wait_ld();
#pragma unroll
          for (int k = 0; k < 32; ++k) o[k] = __float_as_uint(__uint_as_float(o[k]) * alpha);
          ptx::tmem_st_32x32b_x32(t_o + c * 32, o);
        }
      }
      ptx::tcgen05_wait_st();
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->p_full[i & 1]);
    }
    if (ok && nsteps > 0) ok = ptx::mbar_wait(&bars->o_final, 0u, p.timeout_ns, abort_flag);
    if (!ok) {
      if (lane == 0) { fail(p, 3u, 0u, 0u); *abort_flag = 1; }
    } else {
      ptx::tcgen05_fence_after();
      const int64_t grow = static_cast<int64_t>(grow0) + row;
      if (p.splits > 1) {
        // unnormalised partial result of this slice
        float* po = p.part_o + (static_cast<int64_t>(split) * p.total_rows + grow) * kDV + half * kHalf;
        if (row_valid && half == 0) {
          float* ml = p.part_ml + (static_cast<int64_t>(split) * p.total_rows + grow) * 2;
          ml[0] = m_ref; ml[1] = l;
        }
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t o[32];
          if (nsteps > 0) { ptx::tmem_ld_32x32b_x32(t_o + c * 32, o); ptx::tcgen05_wait_ld(); }
          else {
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = 0u;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 8; ++u) ptx::st_global_v4(po + c * 32 + u * 4, make_uint4(o[u * 4], o[u * 4 + 1], o[u * 4 + 2], o[u * 4 + 3]));
          }
        }
      } else {
        const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
        uint8_t* orow = static_cast<uint8_t*>(p.out) + (grow * kDV + half * kHalf) * 2;
#pragma unroll
        for (int c = 0; c < kHalf / 32; ++c) {
          uint32_t o[32];
          if (nsteps > 0) { ptx::tmem_ld_32x32b_x32(t_o + c * 32, o); ptx::tcgen05_wait_ld(); }
          else {
#pragma unroll
            for (int k = 0; k < 32; ++k) o[k] = 0u;
          }
          if (row_valid) {
#pragma unroll
            for (int u = 0; u < 4; ++u) {
              uint32_t w[4];
#pragma unroll
              for (int e = 0; e < 4; ++e)
                w[e] = pack16(__uint_as_float(o[u * 8 + 2 * e]) * inv, __uint_as_float(o[u * 8 + 2 * e + 1]) * inv, p.fmt);
              ptx::st_global_v4(orow + c * 64 + u * 16, make_uint4(w[0], w[1], w[2], w[3]));
            }
          }
        }
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  if (warp == kIssuerWarp) ptx::tmem_dealloc(tmem, kTmemCols);
}

// Merges the slices of a sequence: out = sum_s 2^(m_s - m) O_s / sum_s 2^(m_s - m) l_s. One block per row.
__global__ void mla_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml, void* out,
                                   int total_rows, int splits, int fmt) {
  const int64_t row = blockIdx.x;
  float m = -INFINITY;
  for (int s = 0; s < splits; ++s) m = fmaxf(m, part_ml[(static_cast<int64_t>(s) * total_rows + row) * 2]);
  float L = 0.0f;
  float acc[4] = {0.0f, 0.0f, 0.0f, 0.0f};
  const int col = threadIdx.x * 4;                 // 128 threads x 4 columns
  for (int s = 0; s < splits; ++s) {
    const float* ml = part_ml + (static_cast<int64_t>(s) * total_rows + row) * 2;
    const float wgt = (ml[0] == -INFINITY) ? 0.0f : exp2f(ml[0] - m);
    L += wgt * ml[1];
    const float4 o = *reinterpret_cast<const float4*>(part_o + (static_cast<int64_t>(s) * total_rows + row) * kDV + col);
    acc[0] += wgt * o.x; acc[1] += wgt * o.y; acc[2] += wgt * o.z; acc[3] += wgt * o.w;
  }
  const float inv = L > 0.0f ? 1.0f / L : 0.0f;
  uint2 w;
  w.x = pack16(acc[0] * inv, acc[1] * inv, fmt);
  w.y = pack16(acc[2] * inv, acc[3] * inv, fmt);
  *reinterpret_cast<uint2*>(static_cast<uint8_t*>(out) + (row * kDV + col) * 2) = w;
}

}  // namespace mla
}  // namespace catcoc

using namespace catcoc;
using namespace catcoc::host;

namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// A [pages, rows, cols] array (cols contiguous, 16-bit elements) as a tensor map with a {64, box_rows, ...} box.
// blocks == 1: {cols, rows, pages} (rank 2 when pages == 0). blocks > 1: the columns are cut into `blocks` blocks of
// 64 that become a dimension of their own behind the rows, {64, rows, blocks, pages}, so that one copy lays the
// blocks out one after the other in shared memory.
int encode(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int64_t cols, int64_t rows, int64_t pages, int blocks,
           int box_rows) {
  static EncodeTiledFn fn = driver_fn<EncodeTiledFn>("cuTensorMapEncodeTiled");
  if (fn == nullptr) return CATCOC_E_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) { set_error("mla_decode operands must be 16-byte aligned"); return CATCOC_E_ALIGNMENT; }
  cuuint64_t gdim[4];
  cuuint64_t gstride[3];
  cuuint32_t box[4];
  cuuint32_t estr[4] = {1, 1, 1, 1};
  int rank = 0;
  gdim[rank] = blocks > 1 ? 64 : static_cast<cuuint64_t>(cols); box[rank++] = 64;
  gdim[rank] = static_cast<cuuint64_t>(rows); gstride[rank - 1] = static_cast<cuuint64_t>(cols) * 2; box[rank++] = static_cast<cuuint32_t>(box_rows);
  if (blocks > 1) { gdim[rank] = static_cast<cuuint64_t>(blocks); gstride[rank - 1] = 128; box[rank++] = static_cast<cuuint32_t>(blocks); }
  if (pages > 0) { gdim[rank] = static_cast<cuuint64_t>(pages); gstride[rank - 1] = static_cast<cuuint64_t>(rows) * cols * 2; box[rank++] = 1; }
  CUresult r = fn(tm, dt, static_cast<cuuint32_t>(rank), const_cast<void*>(base), gdim, gstride, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (mla) failed: CUresult %d", static_cast<int>(r)); return CATCOC_E_DRIVER; }
  return CATCOC_OK;
}
}  // namespace

extern "C" int64_t catcoc_mla_workspace_bytes(int B, int q_len, int H, int splits) {
  if (splits <= 1) return 0;
  const int64_t rows = static_cast<int64_t>(B) * q_len * H;
  return static_cast<int64_t>(splits) * rows * (mla::kDV + 2) * static_cast<int64_t>(sizeof(float));
}

extern "C" int catcoc_mla_decode(const void* q_nope, const void* q_rope, const void* ckv, const void* krope,
                                 const int* block_table, const int* kv_lens, void* out, void* workspace, int B, int q_len,
                                 int H, int num_pages, int max_pages, int fmt, int causal, float scale, int splits,
                                 uint32_t* status, uint64_t timeout_ns, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (!q_nope || !q_rope || !ckv || !krope || !block_table || !kv_lens || !out || !status || B <= 0 || H <= 0 ||
      num_pages <= 0 || max_pages <= 0) {
    set_error("mla_decode: bad arguments");
    return CATCOC_E_BAD_ARG;
  }
  if (q_len < 1 || q_len > 4) { set_error("mla_decode: %d new tokens per sequence (1 to 4 are built)", q_len); return CATCOC_E_UNSUPPORTED; }
  if (fmt != CATCOC_FMT_F16 && fmt != CATCOC_FMT_BF16) { set_error("mla_decode takes fp16 / bf16"); return CATCOC_E_UNSUPPORTED; }
  if (!(scale > 0.0f)) { set_error("mla_decode: the softmax scale must be positive"); return CATCOC_E_UNSUPPORTED; }
  if (splits < 1 || splits > 64) { set_error("mla_decode: %d slices per sequence (1 to 64)", splits); return CATCOC_E_BAD_ARG; }
  if (splits > 1 && workspace == nullptr) { set_error("mla_decode: more than one slice needs the workspace"); return CATCOC_E_BAD_ARG; }
  mla::MlaParams p;
  memset(&p, 0, sizeof(p));
  const CUtensorMapDataType dt = fmt == CATCOC_FMT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  const int rows_per_item = q_len * H;
  const int64_t total_rows = static_cast<int64_t>(B) * rows_per_item;
  if (total_rows > (1 << 30)) { set_error("mla_decode: too many query rows"); return CATCOC_E_BAD_ARG; }
  const int qr = rows_per_item <= 64 ? 64 : 128;
  int rc = encode(&p.tm_qn, q_nope, dt, mla::kDV, total_rows, 0, mla::kDV / 64, qr);
  if (rc == 0) rc = encode(&p.tm_qr, q_rope, dt, mla::kDR, total_rows, 0, 1, qr);
  if (rc == 0) rc = encode(&p.tm_kn, ckv, dt, mla::kDV, mla::kPage, num_pages, mla::kDV / 64, mla::kBKV);
  if (rc == 0) rc = encode(&p.tm_kr, krope, dt, mla::kDR, mla::kPage, num_pages, 1, mla::kBKV);
  if (rc != 0) return rc;
  p.block_table = block_table; p.kv_lens = kv_lens; p.out = out;
  p.B = B; p.q_len = q_len; p.H = H; p.max_pages = max_pages; p.num_pages = num_pages; p.splits = splits;
  p.rows_per_item = rows_per_item;
  p.chunks_per_item = (rows_per_item + 127) / 128;
  p.total_rows = static_cast<int>(total_rows);
  if (splits > 1) {
    p.part_o = static_cast<float*>(workspace);
    p.part_ml = p.part_o + static_cast<int64_t>(splits) * total_rows * mla::kDV;
  }
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.fmt = fmt;
  const uint32_t f = fmt == CATCOC_FMT_BF16 ? 1u : 0u;
  p.idesc_qk = ptx::make_instr_desc(1u, f, f, 0u, 0u, 128u, static_cast<uint32_t>(mla::kBKV));
  p.idesc_pv = ptx::make_instr_desc(1u, f, f, 0u, 1u, 128u, static_cast<uint32_t>(mla::kHalf));
  p.status = status;
  p.timeout_ns = timeout_ns ? timeout_ns : 10000000000ull;
  const dim3 grid(2, static_cast<unsigned>(B * p.chunks_per_item), static_cast<unsigned>(splits));
  const int slots = qr == 64 ? 4 : 2;
  const size_t smem = static_cast<size_t>(mla::kChunks) * qr * 128 + static_cast<size_t>(slots) * mla::kSlotBytes + sizeof(mla::Bars) + 1024 + 64;
  if (qr == 64) {
    static cudaError_t once = cudaFuncSetAttribute(mla::mla_decode_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (once != cudaSuccess) { set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(once)); return -1000 - static_cast<int>(once); }
    mla::mla_decode_kernel<64><<<grid, mla::kThreads, smem, stream>>>(p);
  } else {
    static cudaError_t once = cudaFuncSetAttribute(mla::mla_decode_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (once != cudaSuccess) { set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(once)); return -1000 - static_cast<int>(once); }
    mla::mla_decode_kernel<128><<<grid, mla::kThreads, smem, stream>>>(p);
  }
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("mla_decode launch failed: %s", cudaGetErrorString(e)); return -1000 - static_cast<int>(e); }
  if (splits > 1) {
    mla::mla_combine_kernel<<<static_cast<unsigned>(total_rows), 128, 0, stream>>>(p.part_o, p.part_ml, out, p.total_rows, splits, fmt);
    e = cudaGetLastError();
    if (e != cudaSuccess) { set_error("mla_combine launch failed: %s", cudaGetErrorString(e)); return -1000 - static_cast<int>(e); }
  }
  return CATCOC_OK;
}
