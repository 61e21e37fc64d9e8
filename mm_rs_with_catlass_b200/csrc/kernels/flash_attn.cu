// Flash attention forward on tcgen05: one CTA per 256 query rows (two tiles of 128) of one (batch, head).
//
//   warps 0..3  softmax of tile 0 : one query row per thread: tcgen05.ld the scores, row maximum, exp2, row sum,
//   warps 4..7  softmax of tile 1   P (operand dtype) written back over the scores with tcgen05.st, O rescaled in
//                                   TMEM when the running maximum moved by more than 2^8, final O / l and the store
//   warp 8      TMA producer      : both Q tiles once, then K and V blocks of 128 keys through one ring of slots
//   warp 9      MMA issuer        : S_t = Q_t K^T into TMEM, O_t += P_t V with P read from TMEM (the A operand of
//                                   tcgen05.mma may live there), alternating between the two tiles
//
// TMEM columns: S_0 [0, 128), S_1 [128, 256), O_0 [256, 256 + D), O_1 [256 + D, 256 + 2 D); P_t is 64 columns of
// packed 16-bit pairs on top of S_t. While the softmax warps of one tile work, the tensor core runs the other
// tile's two products, so neither waits for the other in the steady state.
//
// The online-softmax recurrence (m: reference maximum, l: running sum, per row, in the log2 domain):
//   P = exp2(scale S - m),  l' = l a + rowsum(P),  O' = O a + P V,  a = exp2(m - m')
// m follows the running maximum lazily: it moves only when some row of the warp exceeds it by more than 8, i.e.
// P stays below 2^8 (exact in fp32, harmless for a 16-bit P), and then O and l are rescaled. Most blocks skip the
// rescale and its trip through TMEM.
//
// Roles of the reference this kernel plays (different construction, same jobs):
//   3rdparty/catlass/include/catlass/gemm/block/block_mmad_fa_qk.hpp, block_mmad_fa_pv.hpp
//   3rdparty/catlass/include/catlass/epilogue/block/block_epilogue_fa_softmax.hpp, ..._fa_rescale_o.hpp
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cstring>
#include "catcoc/capi.h"
#include "catcoc/host_util.h"
#include "catcoc/params.h"
#include "catcoc/ptx.cuh"

namespace catcoc {
namespace attn {

constexpr int kBQ = 128;          // query rows per tile == TMEM lanes
constexpr int kTiles = 2;         // query tiles per CTA
constexpr int kBKV = 128;         // keys per block
constexpr int kThreads = 320;     // 2 x 4 softmax warps, producer, issuer
constexpr int kProducerWarp = 8, kIssuerWarp = 9;
constexpr int kBlockBytes = 128 * 128;   // one 128-row x 128-byte (64 element) swizzled block
constexpr int kMaxSlots = 8;
constexpr float kLazyRescale = 8.0f;     // log2 units the running maximum may exceed the reference by

struct AttnParams {
  CUtensorMap tm_q, tm_k, tm_v;   // {D, S, B * H} with a {64, 128, 1} box, 128-byte swizzle
  void* out;                      // [B, Hq, Sq, D]
  int B, Hq, Hk, Sq, Sk, D;
  int causal;                     // key j is visible to query i when j <= i + (Sk - Sq)
  float scale_log2;               // softmax scale * log2(e), > 0
  int fmt;                        // FMT_F16 or FMT_BF16
  uint32_t idesc_qk, idesc_pv;
  uint32_t* status;
  uint64_t timeout_ns;
};

struct Bars {
  uint64_t q_full, kv_full[kMaxSlots], kv_empty[kMaxSlots], s_full[kTiles], p_full[kTiles], o_done[kTiles];
  uint32_t tmem_base, abort_flag;
};

CATCOC_DEVICE void fail(const AttnParams& p, uint32_t what, uint32_t a, uint32_t b) {
  if (atomicCAS(p.status, 0u, static_cast<uint32_t>(STATUS_TIMEOUT_PIPELINE)) == 0u) {
    p.status[1] = 0u; p.status[2] = 100u + what; p.status[3] = a; p.status[4] = b; p.status[5] = 0u;
    p.status[6] = blockIdx.x;
    __threadfence_system();
  }
}

template <int FMT>
CATCOC_DEVICE uint32_t pack16(float lo, float hi) {
  if constexpr (FMT == FMT_BF16) { __nv_bfloat162 hh = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&hh); }
  else { __half2 hh = __floats2half2_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&hh); }
}

// D: head dimension; FMT: operand and output dtype (compile time: the softmax loop packs 64 pairs per row and block)
template <int D, int FMT>
__global__ void __launch_bounds__(kThreads, 1) flash_attn_kernel(const __grid_constant__ AttnParams p) {
  constexpr int kDB = D / 64;                    // 128-byte blocks along the head dimension
  constexpr int kQBytes = kDB * kBlockBytes;     // one Q tile
  constexpr int kSlotBytes = kDB * kBlockBytes;  // one K or V block: 128 keys x D
  constexpr int kSlots = D == 128 ? 4 : 8;       // ring of K / V blocks (K_0 V_0 K_1 V_1 ...)
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kOCol = 256;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;                            // two Q tiles
  uint8_t* skv = sq + kTiles * kQBytes;
  Bars* bars = reinterpret_cast<Bars*>(skv + kSlots * kSlotBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qt = static_cast<int>(gridDim.x) - 1 - static_cast<int>(blockIdx.x);   // late (long) causal tiles first
  const int q0 = qt * (kTiles * kBQ);
  const int bh = blockIdx.y;                       // b * Hq + h
  const int b = bh / p.Hq, h = bh - b * p.Hq;
  const int bhk = b * p.Hk + h / (p.Hq / p.Hk);    // grouped-query attention: several query heads share one KV head
  const int shift = p.Sk - p.Sq;                   // causal diagonal offset
  // key blocks each tile walks (tile 1 never fewer than tile 0; rows past Sq are computed and not stored)
  int nblk[kTiles];
#pragma unroll
  for (int t = 0; t < kTiles; ++t) {
    const int kv_end = p.causal ? min(p.Sk, q0 + (t + 1) * kBQ + shift) : p.Sk;
    nblk[t] = (kv_end + kBKV - 1) / kBKV;
  }
  const int nmax = nblk[1];

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kSlots; ++s) { ptx::mbar_init(&bars->kv_full[s], 1); ptx::mbar_init(&bars->kv_empty[s], 1); }
    for (int t = 0; t < kTiles; ++t) {
      ptx::mbar_init(&bars->s_full[t], 1);
      ptx::mbar_init(&bars->p_full[t], 4);         // one arrival per softmax warp
      ptx::mbar_init(&bars->o_done[t], 1);
    }
    bars->abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&p.tm_q); ptx::prefetch_tmap(&p.tm_k); ptx::prefetch_tmap(&p.tm_v);
  }
  if (warp == kIssuerWarp) { ptx::tmem_alloc(&bars->tmem_base, kTmemCols); ptx::tmem_relinquish(); }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == kProducerWarp) {
    // ------------------------------ TMA producer ------------------------------
    if (ptx::elect_one()) {
      ptx::mbar_expect_tx(&bars->q_full, kTiles * kQBytes);
      for (int t = 0; t < kTiles; ++t)
        for (int d = 0; d < kDB; ++d)
          ptx::tma_load_3d(sq + t * kQBytes + d * kBlockBytes, &p.tm_q, &bars->q_full, d * 64, q0 + t * kBQ, bh);
    }
    __syncwarp();
    // item 2 j is K block j, item 2 j + 1 is V block j; item i lives in slot i % kSlots
    for (int item = 0; item < 2 * nmax; ++item) {
      const int slot = item % kSlots;
      const uint32_t use = static_cast<uint32_t>(item / kSlots);
      if (!ptx::mbar_wait(&bars->kv_empty[slot], (use & 1u) ^ 1u, p.timeout_ns, abort_flag)) {
        if (lane == 0) { fail(p, 1u, item, 0u); *abort_flag = 1; }
        break;
      }
      if (ptx::elect_one()) {
        ptx::mbar_expect_tx(&bars->kv_full[slot], kSlotBytes);
        const CUtensorMap* tm = (item & 1) ? &p.tm_v : &p.tm_k;
        for (int d = 0; d < kDB; ++d)
          ptx::tma_load_3d(skv + slot * kSlotBytes + d * kBlockBytes, tm, &bars->kv_full[slot], d * 64, (item >> 1) * kBKV, bhk);
      }
      __syncwarp();
    }
  } else if (warp == kIssuerWarp) {
    // ------------------------------ MMA issuer ------------------------------
    auto wait_item = [&](int item) {
      return ptx::mbar_wait(&bars->kv_full[item % kSlots], static_cast<uint32_t>(item / kSlots) & 1u, p.timeout_ns, abort_flag);
    };
    auto issue_qk = [&](int t, int item) {
      // S_t[128, 128 keys] = Q_t[128, D] K^T: both operands K-major (D contiguous), 16 elements of D per MMA
      const uint64_t dq = ptx::make_smem_desc_sw128(ptx::smem_u32(sq + t * kQBytes), 16u, 1024u);
      const uint64_t dk = ptx::make_smem_desc_sw128(ptx::smem_u32(skv + (item % kSlots) * kSlotBytes), 16u, 1024u);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4);
        ptx::umma_f16(tmem + t * 128, dq + off, dk + off, p.idesc_qk, kk != 0 ? 1u : 0u);
      }
      ptx::tcgen05_commit(&bars->s_full[t]);
    };
    auto issue_pv = [&](int t, int item, bool accumulate) {
      // O_t[128, D] += P_t[128, 128 keys] V[128 keys, D]: P from TMEM (row = lane, two keys per 32-bit column, 8
      // columns per MMA), V MN-major (D contiguous): 16 key rows per MMA = 2048 bytes down a block, blocks of 64
      // head-dim columns 16 KiB apart
      const uint64_t dv = ptx::make_smem_desc_sw128(ptx::smem_u32(skv + (item % kSlots) * kSlotBytes),
                                                    static_cast<uint32_t>(kBlockBytes), 1024u);
#pragma unroll
      for (int kk = 0; kk < kBKV / 16; ++kk) {
        const uint64_t offb = static_cast<uint64_t>((kk * 16 * 128) >> 4);
        ptx::umma_f16_ts(tmem + kOCol + t * D, tmem + t * 128 + kk * 8, dv + offb, p.idesc_pv, (accumulate || kk != 0) ? 1u : 0u);
      }
    };
    bool ok = ptx::mbar_wait(&bars->q_full, 0u, p.timeout_ns, abort_flag);
    if (ok) ok = wait_item(0);
    if (ok) {
      ptx::tcgen05_fence_after();
      if (ptx::elect_one()) {
        issue_qk(0, 0);
        issue_qk(1, 0);
        ptx::tcgen05_commit(&bars->kv_empty[0]);
      }
      __syncwarp();
    }
    for (int j = 0; ok && j < nmax; ++j) {
      const int v_item = 2 * j + 1, k_next = 2 * j + 2;
      const bool next0 = j + 1 < nblk[0], next1 = j + 1 < nblk[1];
      bool v_here = false;
      if (j < nblk[0]) {
        // P_0(j) is in TMEM and O_0 has been rescaled
        ok = ptx::mbar_wait(&bars->p_full[0], static_cast<uint32_t>(j & 1), p.timeout_ns, abort_flag) && wait_item(v_item);
        if (!ok) break;
        v_here = true;
        ptx::tcgen05_fence_after();
        if (ptx::elect_one()) {
          issue_pv(0, v_item, j > 0);
          if (!next0) ptx::tcgen05_commit(&bars->o_done[0]);
        }
        __syncwarp();
        if (next0) {
          ok = wait_item(k_next);
          if (!ok) break;
          ptx::tcgen05_fence_after();
          if (ptx::elect_one()) issue_qk(0, k_next);      // the scores of block j + 1 land on P_0(j): in issue order
          __syncwarp();
        }
      }
      ok = ptx::mbar_wait(&bars->p_full[1], static_cast<uint32_t>(j & 1), p.timeout_ns, abort_flag) && (v_here || wait_item(v_item));
      if (!ok) break;
      ptx::tcgen05_fence_after();
      if (ptx::elect_one()) {
        issue_pv(1, v_item, j > 0);
        ptx::tcgen05_commit(&bars->kv_empty[v_item % kSlots]);
        if (!next1) ptx::tcgen05_commit(&bars->o_done[1]);
      }
      __syncwarp();
      if (next1) {
        ok = wait_item(k_next);
        if (!ok) break;
        ptx::tcgen05_fence_after();
        if (ptx::elect_one()) {
          issue_qk(1, k_next);
          ptx::tcgen05_commit(&bars->kv_empty[k_next % kSlots]);
        }
        __syncwarp();
      }
    }
    if (!ok && lane == 0) { fail(p, 2u, 0u, 0u); *abort_flag = 1; }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int t = warp >> 2;                         // query tile of this warp
    const int qd = warp & 3;                         // TMEM lane quarter of this warp
    const int row = qd * 32 + lane;                  // query row inside the tile
    const int qi = q0 + t * kBQ + row;
    const uint32_t t_s = tmem + (static_cast<uint32_t>(qd * 32) << 16) + t * 128;   // scores, and P on top of them
    const uint32_t t_o = tmem + (static_cast<uint32_t>(qd * 32) << 16) + kOCol + t * D;
    const int n_mine = nblk[t];
    const int vis = p.causal ? min(p.Sk, qi + shift + 1) : p.Sk;            // keys [0, vis) are visible to this row
    const int vis_tile = p.causal ? min(p.Sk, q0 + t * kBQ + shift + 1) : p.Sk;   // ... to every row of the tile
    const float sc = p.scale_log2;
    float m_ref = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < n_mine; ++j) {
      if (!ptx::mbar_wait(&bars->s_full[t], static_cast<uint32_t>(j & 1), p.timeout_ns, abort_flag)) { ok = false; break; }
      ptx::tcgen05_fence_after();
      const int key0 = j * kBKV;
      const bool masked = key0 + kBKV > vis_tile;    // some row of the tile does not see all of this block
      // pass 1: row maximum of the raw scores (the scale is positive)
      float mx = -INFINITY;
#pragma unroll
      for (int c = 0; c < kBKV / 64; ++c) {
        uint32_t v0[32], v1[32];
        ptx::tmem_ld_32x32b_x32(t_s + c * 64, v0);
        ptx::tmem_ld_32x32b_x32(t_s + c * 64 + 32, v1);
        ptx::tcgen05_wait_ld();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            if (key0 + c * 64 + i < vis) mx = fmaxf(mx, __uint_as_float(v0[i]));
            if (key0 + c * 64 + 32 + i < vis) mx = fmaxf(mx, __uint_as_float(v1[i]));
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, fmaxf(__uint_as_float(v0[i]), __uint_as_float(v1[i])));
        }
      }
      const float m_new = fmaxf(m_ref, mx * sc);
      const bool move = __any_sync(0xffffffffu, m_new > m_ref + kLazyRescale);   // -inf + 8 = -inf: the first block moves
      const float m_use = move ? m_new : m_ref;
      const float m_safe = (m_use == -INFINITY) ? 0.0f : m_use;                   // a row that sees nothing yet
      const float alpha = !move ? 1.0f : ((m_ref == -INFINITY) ? 0.0f : ptx::ex2_approx(m_ref - m_safe));
      // pass 2: P = exp2(scale S - m), its row sum, P packed over the scores it came from
      float sum = 0.0f;
#pragma unroll
      for (int c = 0; c < kBKV / 32; ++c) {
        uint32_t v[32], w[16];
        ptx::tmem_ld_32x32b_x32(t_s + c * 32, v);
        ptx::tcgen05_wait_ld();
        if (masked) {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = (key0 + c * 32 + i < vis) ? ptx::ex2_approx(fmaf(__uint_as_float(v[i]), sc, -m_safe)) : 0.0f;
            const float e1 = (key0 + c * 32 + i + 1 < vis) ? ptx::ex2_approx(fmaf(__uint_as_float(v[i + 1]), sc, -m_safe)) : 0.0f;
            sum += e0 + e1;
            w[i >> 1] = pack16<FMT>(e0, e1);
          }
        } else {
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            const float e0 = ptx::ex2_approx(fmaf(__uint_as_float(v[i]), sc, -m_safe));
            const float e1 = ptx::ex2_approx(fmaf(__uint_as_float(v[i + 1]), sc, -m_safe));
            sum += e0 + e1;
            w[i >> 1] = pack16<FMT>(e0, e1);
          }
        }
        ptx::tmem_st_32x32b_x16(t_s + c * 16, w);
      }
      l = l * alpha + sum;
      m_ref = m_use;
      // O *= alpha where the reference maximum moved. s_full(j) was committed behind P V of block j - 1, so O is whole.
      if (move && j > 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(t_o + c * 32, v);
          ptx::tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          ptx::tmem_st_32x32b_x32(t_o + c * 32, v);
        }
      }
      ptx::tcgen05_wait_st();
      ptx::tcgen05_fence_before();
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->p_full[t]);
    }
    if (ok) ok = ptx::mbar_wait(&bars->o_done[t], 0u, p.timeout_ns, abort_flag);
    if (!ok) {
      if (lane == 0) { fail(p, 3u, t, 0u); *abort_flag = 1; }
    } else {
      ptx::tcgen05_fence_after();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      uint8_t* orow = static_cast<uint8_t*>(p.out) + (static_cast<int64_t>(bh) * p.Sq + qi) * D * 2;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(t_o + c * 32, v);
        ptx::tcgen05_wait_ld();
        if (qi < p.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e)
              w[e] = pack16<FMT>(__uint_as_float(v[u * 8 + 2 * e]) * inv, __uint_as_float(v[u * 8 + 2 * e + 1]) * inv);
            ptx::st_global_v4(orow + c * 64 + u * 16, make_uint4(w[0], w[1], w[2], w[3]));
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

}  // namespace attn
}  // namespace catcoc

using namespace catcoc;
using namespace catcoc::host;

namespace {
using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

// [BH, S, D] (D contiguous) as {D, S, BH} with a {64, 128, 1} box: rows past S read as zeros
int encode_bsd(CUtensorMap* tm, const void* base, CUtensorMapDataType dt, int64_t BH, int64_t S, int64_t D) {
  static EncodeTiledFn fn = driver_fn<EncodeTiledFn>("cuTensorMapEncodeTiled");
  if (fn == nullptr) return CATCOC_E_DRIVER;
  if (reinterpret_cast<uintptr_t>(base) & 15) { set_error("attention operands must be 16-byte aligned"); return CATCOC_E_ALIGNMENT; }
  cuuint64_t gdim[3] = {static_cast<cuuint64_t>(D), static_cast<cuuint64_t>(S), static_cast<cuuint64_t>(BH)};
  cuuint64_t gstride[2] = {static_cast<cuuint64_t>(D) * 2, static_cast<cuuint64_t>(S) * D * 2};
  cuuint32_t box[3] = {64, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(tm, dt, 3, const_cast<void*>(base), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) { set_error("cuTensorMapEncodeTiled (attention) failed: CUresult %d", static_cast<int>(r)); return CATCOC_E_DRIVER; }
  return CATCOC_OK;
}
}  // namespace

extern "C" int catcoc_flash_attention(const void* q, const void* k, const void* v, void* out, int B, int Hq, int Hk,
                                      int Sq, int Sk, int D, int fmt, int causal, float scale, uint32_t* status,
                                      uint64_t timeout_ns, void* stream) {
  if (!q || !k || !v || !out || !status || B <= 0 || Hq <= 0 || Hk <= 0 || Sq <= 0 || Sk <= 0) {
    set_error("flash_attention: bad arguments");
    return CATCOC_E_BAD_ARG;
  }
  if (D != 64 && D != 128) { set_error("flash_attention: head dimension %d (64 and 128 are built)", D); return CATCOC_E_UNSUPPORTED; }
  if (Hq % Hk != 0) { set_error("flash_attention: %d query heads do not divide over %d key / value heads", Hq, Hk); return CATCOC_E_BAD_ARG; }
  if (fmt != CATCOC_FMT_F16 && fmt != CATCOC_FMT_BF16) { set_error("flash_attention takes fp16 / bf16"); return CATCOC_E_UNSUPPORTED; }
  if (causal && Sk < Sq) { set_error("causal attention needs Sk >= Sq"); return CATCOC_E_BAD_ARG; }
  if (!(scale > 0.0f)) { set_error("flash_attention: the softmax scale must be positive (the row maximum is taken before scaling)"); return CATCOC_E_UNSUPPORTED; }
  attn::AttnParams p;
  memset(&p, 0, sizeof(p));
  const CUtensorMapDataType dt = fmt == CATCOC_FMT_F16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  int rc = encode_bsd(&p.tm_q, q, dt, static_cast<int64_t>(B) * Hq, Sq, D);
  if (rc == 0) rc = encode_bsd(&p.tm_k, k, dt, static_cast<int64_t>(B) * Hk, Sk, D);
  if (rc == 0) rc = encode_bsd(&p.tm_v, v, dt, static_cast<int64_t>(B) * Hk, Sk, D);
  if (rc != 0) return rc;
  p.out = out;
  p.B = B; p.Hq = Hq; p.Hk = Hk; p.Sq = Sq; p.Sk = Sk; p.D = D;
  p.causal = causal ? 1 : 0;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.fmt = fmt;
  const uint32_t f = fmt == CATCOC_FMT_BF16 ? 1u : 0u;
  p.idesc_qk = ptx::make_instr_desc(1u, f, f, 0u, 0u, 128u, 128u);
  p.idesc_pv = ptx::make_instr_desc(1u, f, f, 0u, 1u, 128u, static_cast<uint32_t>(D));
  p.status = status;
  p.timeout_ns = timeout_ns ? timeout_ns : 10000000000ull;
  const int rows = attn::kTiles * attn::kBQ;
  const dim3 grid((Sq + rows - 1) / rows, B * Hq, 1);
  const int db = D / 64;
  const int slots = D == 128 ? 4 : 8;
  const size_t smem = static_cast<size_t>(attn::kTiles * db + slots * db) * attn::kBlockBytes + sizeof(attn::Bars) + 1024 + 64;
  cudaError_t e;
  auto launch = [&](auto kernel) -> int {
    // (one attribute call per launch: it is cheap and keeps the four instantiations in one place)
    cudaError_t a = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (a != cudaSuccess) { set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(a)); return -1000 - static_cast<int>(a); }
    kernel<<<grid, attn::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
    return 0;
  };
  int lrc;
  if (D == 128) lrc = fmt == CATCOC_FMT_BF16 ? launch(attn::flash_attn_kernel<128, FMT_BF16>) : launch(attn::flash_attn_kernel<128, FMT_F16>);
  else lrc = fmt == CATCOC_FMT_BF16 ? launch(attn::flash_attn_kernel<64, FMT_BF16>) : launch(attn::flash_attn_kernel<64, FMT_F16>);
  if (lrc != 0) return lrc;
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("flash_attention launch failed: %s", cudaGetErrorString(e)); return -1000 - static_cast<int>(e); }
  return CATCOC_OK;
}
