// Flash attention forward on tcgen05: one CTA per 128 query rows of one (batch, head).
//
//   warp 0      TMA producer : Q tile once, then K and V blocks of 128 keys into a 2-stage ring
//   warp 1      MMA issuer   : S = Q K^T into TMEM columns [0, 128), O += P V into [128, 128 + D)
//   warps 2..5  softmax      : one query row per thread: tcgen05.ld the scores, scale / mask, running
//                              max and sum, P (operand dtype) into shared memory as the A operand of
//                              the second product, rescale of O in TMEM (tcgen05.ld / st) when the
//                              running max moved, final O / l and the store
//
// The online-softmax recurrence is the usual one (m: running max, l: running sum, both per row):
//   m' = max(m, rowmax(S)),  P = exp2(S - m'),  l' = l * exp2(m - m') + rowsum(P),  O' = O * exp2(m - m') + P V
// with S pre-multiplied by scale * log2(e). QK^T of block j+1 is issued right behind P V of block j,
// so the tensor core works on the next scores while the softmax warps finish the current block.
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

constexpr int kBQ = 128;          // query rows per CTA == TMEM lanes
constexpr int kBKV = 128;         // keys per block
constexpr int kThreads = 192;     // producer, issuer, 4 softmax warps
constexpr int kBlockBytes = 128 * 128;   // one 128-row x 128-byte (64 element) swizzled block
constexpr int kStages = 2;

struct AttnParams {
  CUtensorMap tm_q, tm_k, tm_v;   // {D, S, B * H} with a {64, 128, 1} box, 128-byte swizzle
  void* out;                      // [B, Hq, Sq, D]
  int B, Hq, Hk, Sq, Sk, D;
  int causal;                     // key j is visible to query i when j <= i + (Sk - Sq)
  float scale_log2;               // softmax scale * log2(e)
  int fmt;                        // FMT_F16 or FMT_BF16
  uint32_t idesc_qk, idesc_pv;
  uint32_t* status;
  uint64_t timeout_ns;
};

struct Bars {
  uint64_t q_full, kv_full[kStages], kv_empty[kStages], s_full, p_full, o_done;
  uint32_t tmem_base, abort_flag;
};

CATCOC_DEVICE void fail(const AttnParams& p, uint32_t what, uint32_t a, uint32_t b) {
  if (atomicCAS(p.status, 0u, static_cast<uint32_t>(STATUS_TIMEOUT_PIPELINE)) == 0u) {
    p.status[1] = 0u; p.status[2] = 100u + what; p.status[3] = a; p.status[4] = b; p.status[5] = 0u;
    p.status[6] = blockIdx.x;
    __threadfence_system();
  }
}

template <int D>
__global__ void __launch_bounds__(kThreads, 1) flash_attn_kernel(const __grid_constant__ AttnParams p) {
  constexpr int kDB = D / 64;                    // 128-byte blocks along the head dimension
  constexpr int kQBytes = kDB * kBlockBytes;
  constexpr int kKBytes = kDB * kBlockBytes;     // K block: 128 keys x D
  constexpr int kVBytes = kDB * kBlockBytes;     // V block: 128 keys x D
  constexpr int kPBytes = 2 * kBlockBytes;       // P: 128 rows x 128 keys
  constexpr uint32_t kTmemCols = 256;
  constexpr uint32_t kOCol = 128;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* sq = smem;
  uint8_t* sk = sq + kQBytes;
  uint8_t* sv = sk + kStages * kKBytes;
  uint8_t* sp = sv + kStages * kVBytes;
  Bars* bars = reinterpret_cast<Bars*>(sp + kPBytes);
  volatile uint32_t* abort_flag = &bars->abort_flag;

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kBQ;
  const int bh = blockIdx.y;                       // b * Hq + h
  const int b = bh / p.Hq, h = bh - b * p.Hq;
  const int bhk = b * p.Hk + h / (p.Hq / p.Hk);    // grouped-query attention: several query heads share one KV head
  const int shift = p.Sk - p.Sq;                   // causal diagonal offset
  // keys this query tile can see at all
  int kv_end = p.Sk;
  if (p.causal) kv_end = min(p.Sk, q0 + kBQ + shift);
  const int nblk = kv_end > 0 ? (kv_end + kBKV - 1) / kBKV : 0;

  if (threadIdx.x == 0) {
    ptx::mbar_init(&bars->q_full, 1);
    for (int s = 0; s < kStages; ++s) { ptx::mbar_init(&bars->kv_full[s], 1); ptx::mbar_init(&bars->kv_empty[s], 1); }
    ptx::mbar_init(&bars->s_full, 1);
    ptx::mbar_init(&bars->p_full, 4);              // one arrival per softmax warp
    ptx::mbar_init(&bars->o_done, 1);
    bars->abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::prefetch_tmap(&p.tm_q); ptx::prefetch_tmap(&p.tm_k); ptx::prefetch_tmap(&p.tm_v);
  }
  if (warp == 1) { ptx::tmem_alloc(&bars->tmem_base, kTmemCols); ptx::tmem_relinquish(); }
  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  const uint32_t tmem = bars->tmem_base;

  if (warp == 0) {
    // ------------------------------ TMA producer ------------------------------
    if (ptx::elect_one()) {
      ptx::mbar_expect_tx(&bars->q_full, kQBytes);
      for (int d = 0; d < kDB; ++d) ptx::tma_load_3d(sq + d * kBlockBytes, &p.tm_q, &bars->q_full, d * 64, q0, bh);
    }
    __syncwarp();
    uint32_t phase = 0;
    int st = 0;
    for (int j = 0; j < nblk; ++j) {
      if (!ptx::mbar_wait(&bars->kv_empty[st], phase ^ 1u, p.timeout_ns, abort_flag)) {
        if (lane == 0) { fail(p, 1u, j, 0u); *abort_flag = 1; }
        break;
      }
      if (ptx::elect_one()) {
        ptx::mbar_expect_tx(&bars->kv_full[st], kKBytes + kVBytes);
        for (int d = 0; d < kDB; ++d) {
          ptx::tma_load_3d(sk + st * kKBytes + d * kBlockBytes, &p.tm_k, &bars->kv_full[st], d * 64, j * kBKV, bhk);
          ptx::tma_load_3d(sv + st * kVBytes + d * kBlockBytes, &p.tm_v, &bars->kv_full[st], d * 64, j * kBKV, bhk);
        }
      }
      __syncwarp();
      if (++st == kStages) { st = 0; phase ^= 1u; }
    }
  } else if (warp == 1) {
    // ------------------------------ MMA issuer ------------------------------
    const uint64_t dq = ptx::make_smem_desc_sw128(ptx::smem_u32(sq), 16u, 1024u);
    const uint64_t dp = ptx::make_smem_desc_sw128(ptx::smem_u32(sp), 16u, 1024u);
    auto issue_qk = [&](int st) {
      // S[128, 128 keys] = Q[128, D] K^T: both operands K-major (D contiguous), 16 elements of D per MMA
      const uint64_t dk = ptx::make_smem_desc_sw128(ptx::smem_u32(sk + st * kKBytes), 16u, 1024u);
#pragma unroll
      for (int kk = 0; kk < D / 16; ++kk) {
        const uint64_t off = static_cast<uint64_t>(((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4);
        ptx::umma_f16(tmem, dq + off, dk + off, p.idesc_qk, kk != 0 ? 1u : 0u);
      }
      ptx::tcgen05_commit(&bars->s_full);
    };
    auto issue_pv = [&](int st, bool accumulate) {
      // O[128, D] += P[128, 128 keys] V[128 keys, D]: P K-major (keys contiguous), V MN-major (D contiguous):
      // 16 key rows per MMA = 2048 bytes down a block, blocks of 64 head-dim columns 16 KiB apart
      const uint64_t dv = ptx::make_smem_desc_sw128(ptx::smem_u32(sv + st * kVBytes), static_cast<uint32_t>(kBlockBytes), 1024u);
#pragma unroll
      for (int kk = 0; kk < kBKV / 16; ++kk) {
        const uint64_t offa = static_cast<uint64_t>(((kk >> 2) * kBlockBytes + (kk & 3) * 32) >> 4);
        const uint64_t offb = static_cast<uint64_t>((kk * 16 * 128) >> 4);
        ptx::umma_f16(tmem + kOCol, dp + offa, dv + offb, p.idesc_pv, (accumulate || kk != 0) ? 1u : 0u);
      }
      ptx::tcgen05_commit(&bars->kv_empty[st]);
      ptx::tcgen05_commit(&bars->o_done);
    };
    bool ok = ptx::mbar_wait(&bars->q_full, 0u, p.timeout_ns, abort_flag);
    uint32_t kv_phase = 0;
    int st = 0;
    if (ok && nblk > 0) {
      ok = ptx::mbar_wait(&bars->kv_full[0], 0u, p.timeout_ns, abort_flag);
      ptx::tcgen05_fence_after();
      if (ok && ptx::elect_one()) issue_qk(0);
      __syncwarp();
    }
    for (int j = 0; ok && j < nblk; ++j) {
      // P(j) is in shared memory and O has been rescaled
      ok = ptx::mbar_wait(&bars->p_full, static_cast<uint32_t>(j & 1), p.timeout_ns, abort_flag);
      if (!ok) break;
      ptx::tcgen05_fence_after();
      if (ptx::elect_one()) issue_pv(st, j > 0);
      __syncwarp();
      int nst = st + 1;
      uint32_t nphase = kv_phase;
      if (nst == kStages) { nst = 0; nphase ^= 1u; }
      if (j + 1 < nblk) {
        ok = ptx::mbar_wait(&bars->kv_full[nst], nphase, p.timeout_ns, abort_flag);
        if (!ok) break;
        ptx::tcgen05_fence_after();
        if (ptx::elect_one()) issue_qk(nst);   // the scores of block j+1 (S was read out before p_full(j))
        __syncwarp();
      }
      st = nst; kv_phase = nphase;
    }
    if (!ok && lane == 0) { fail(p, 2u, 0u, 0u); *abort_flag = 1; }
  } else {
    // ------------------------------ softmax / correction / epilogue ------------------------------
    const int qd = warp & 3;                         // TMEM lane quarter of this warp
    const int row = qd * 32 + lane;                  // query row inside the tile
    const int qi = q0 + row;
    const uint32_t t_s = tmem + (static_cast<uint32_t>(qd * 32) << 16);
    const uint32_t t_o = t_s + kOCol;
    const uint32_t sp_row = ptx::smem_u32(sp) + row * 128;
    float m = -INFINITY, l = 0.0f;
    bool ok = true;
    for (int j = 0; j < nblk; ++j) {
      if (!ptx::mbar_wait(&bars->s_full, static_cast<uint32_t>(j & 1), p.timeout_ns, abort_flag)) { ok = false; break; }
      ptx::tcgen05_fence_after();
      float s[kBKV];
#pragma unroll
      for (int c = 0; c < kBKV / 32; ++c) {
        uint32_t v[32];
        ptx::tmem_ld_32x32b_x32(t_s + c * 32, v);
        ptx::tcgen05_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) s[c * 32 + i] = __uint_as_float(v[i]);
      }
      // scale, mask (keys past the sequence, keys above the causal diagonal), row maximum
      const int key0 = j * kBKV;
      const int vis = p.causal ? min(p.Sk, qi + shift + 1) : p.Sk;    // keys [0, vis) are visible to this row
      float mx = m;
#pragma unroll
      for (int i = 0; i < kBKV; ++i) {
        s[i] = (key0 + i < vis) ? s[i] * p.scale_log2 : -INFINITY;
        mx = fmaxf(mx, s[i]);
      }
      const float m_use = (mx == -INFINITY) ? 0.0f : mx;              // a row that sees nothing yet
      const float alpha = exp2f(m - m_use);                             // 0 on the first block (m = -inf)
      float sum = 0.0f;
#pragma unroll
      for (int i = 0; i < kBKV; ++i) { s[i] = exp2f(s[i] - m_use); sum += s[i]; }
      l = l * alpha + sum;
      m = mx;
      // P V of the previous block must be done with P's shared memory and with O
      if (j > 0) {
        if (!ptx::mbar_wait(&bars->o_done, static_cast<uint32_t>((j - 1) & 1), p.timeout_ns, abort_flag)) { ok = false; break; }
        ptx::tcgen05_fence_after();
      }
      // P as the A operand of the second product: K-major, 128-byte swizzle (16-byte unit u of row r at u ^ (r & 7))
#pragma unroll
      for (int c = 0; c < kBKV / 8; ++c) {
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          if (p.fmt == FMT_BF16) {
            __nv_bfloat162 hh = __floats2bfloat162_rn(s[c * 8 + 2 * e], s[c * 8 + 2 * e + 1]);
            w[e] = *reinterpret_cast<uint32_t*>(&hh);
          } else {
            __half2 hh = __floats2half2_rn(s[c * 8 + 2 * e], s[c * 8 + 2 * e + 1]);
            w[e] = *reinterpret_cast<uint32_t*>(&hh);
          }
        }
        ptx::st_shared_v4(sp_row + (c >> 3) * kBlockBytes + (((c & 7) ^ (row & 7)) << 4), make_uint4(w[0], w[1], w[2], w[3]));
      }
      // O *= alpha where the running maximum moved
      if (j > 0) {
#pragma unroll
        for (int c = 0; c < D / 32; ++c) {
          uint32_t v[32];
          ptx::tmem_ld_32x32b_x32(t_o + c * 32, v);
          ptx::tcgen05_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = __float_as_uint(__uint_as_float(v[i]) * alpha);
          ptx::tmem_st_32x32b_x32(t_o + c * 32, v);
        }
        ptx::tcgen05_wait_st();
      }
      ptx::tcgen05_fence_before();
      ptx::fence_proxy_async_smem();      // P becomes visible to the tensor core's reads of shared memory
      __syncwarp();
      if (lane == 0) ptx::mbar_arrive(&bars->p_full);
    }
    if (ok && nblk > 0) ok = ptx::mbar_wait(&bars->o_done, static_cast<uint32_t>((nblk - 1) & 1), p.timeout_ns, abort_flag);
    if (!ok) {
      if (lane == 0) { fail(p, 3u, 0u, 0u); *abort_flag = 1; }
    } else {
      ptx::tcgen05_fence_after();
      const float inv = (l > 0.0f) ? 1.0f / l : 0.0f;
      uint8_t* orow = static_cast<uint8_t*>(p.out) + (static_cast<int64_t>(bh) * p.Sq + qi) * D * 2;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        if (nblk > 0) { ptx::tmem_ld_32x32b_x32(t_o + c * 32, v); ptx::tcgen05_wait_ld(); }
        else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0u;
        }
        if (qi < p.Sq) {
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const float a = __uint_as_float(v[u * 8 + 2 * e]) * inv, bb = __uint_as_float(v[u * 8 + 2 * e + 1]) * inv;
              if (p.fmt == FMT_BF16) { __nv_bfloat162 hh = __floats2bfloat162_rn(a, bb); w[e] = *reinterpret_cast<uint32_t*>(&hh); }
              else { __half2 hh = __floats2half2_rn(a, bb); w[e] = *reinterpret_cast<uint32_t*>(&hh); }
            }
            ptx::st_global_v4(orow + c * 64 + u * 16, make_uint4(w[0], w[1], w[2], w[3]));
          }
        }
      }
    }
  }

  ptx::tcgen05_fence_before();
  __syncthreads();
  ptx::tcgen05_fence_after();
  if (warp == 1) ptx::tmem_dealloc(tmem, kTmemCols);
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
  const dim3 grid((Sq + attn::kBQ - 1) / attn::kBQ, B * Hq, 1);
  const int db = D / 64;
  const size_t smem = static_cast<size_t>(db + 2 * attn::kStages * db + 2) * attn::kBlockBytes + sizeof(attn::Bars) + 1024 + 64;
  cudaError_t e;
  if (D == 128) {
    static cudaError_t once = cudaFuncSetAttribute(attn::flash_attn_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (once != cudaSuccess) { set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(once)); return -1000 - static_cast<int>(once); }
    attn::flash_attn_kernel<128><<<grid, attn::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  } else {
    static cudaError_t once = cudaFuncSetAttribute(attn::flash_attn_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (once != cudaSuccess) { set_error("cudaFuncSetAttribute failed: %s", cudaGetErrorString(once)); return -1000 - static_cast<int>(once); }
    attn::flash_attn_kernel<64><<<grid, attn::kThreads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  }
  e = cudaGetLastError();
  if (e != cudaSuccess) { set_error("flash_attention launch failed: %s", cudaGetErrorString(e)); return -1000 - static_cast<int>(e); }
  return CATCOC_OK;
}
