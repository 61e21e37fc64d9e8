// Collectives for products with few output tiles and a long K (M up to a few hundred rows). First, the all-reduce /
// reduce-scatter: the second half of a two-launch path. The first launch is the GEMM kernel in its split-K form (K slices as the groups of one launch, fp32
// partial planes in a local workspace), so that every SM streams a share of B. This kernel then
//   phase A  sums the planes of a chunk, rounds to the operand dtype, stores the chunk into this rank's symmetric
//            buffer and stamps (chunk, rank) on every rank (one multimem.st through the switch, or a store per peer);
//   phase B  waits for the W stamps of a chunk of its output rows (all rows for an all-reduce, its own share for a
//            reduce-scatter) and reads the sum of all ranks' copies through the switch
//            (multimem.ld_reduce, fp32 accumulation) or, without a multicast mapping, from the peers in rank order,
//            and writes this rank's output. Every rank reduces every chunk itself: no broadcast, no second hop.
// A one-wave GEMM has nothing to overlap a collective with, so at these sizes the fused tile loop buys nothing and
// costs SMs: with M = 128 and N = 8192 it runs 64 to 128 CTAs that each stream the whole of A.
//
// Protocol: the same epoch stamps as the fused kernel. The launch's epoch is *epoch_ptr + 1; the last CTA to finish
// advances *epoch_ptr unless a wait ran out. The symmetric buffer has two parity halves; the host passes the half of
// this epoch. A rank can start epoch e + 2 (which overwrites the half of epoch e) only after every peer has stamped
// epoch e + 1, i.e. after every peer has finished reading epoch e. Every wait is bounded.
//
// Role in the reference: the small-M end of include/catcoc/dgemm/kernel/matmul_allreduce.hpp, which the reference
// covers with its commInterval knob (examples/dynamic_tiling/include/tiling.h:19-22).
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include "catcoc/capi.h"
#include "catcoc/host_util.h"
#include "catcoc/params.h"
#include "catcoc/ptx.cuh"

namespace catcoc {
namespace {

constexpr int kThreads = 256;
constexpr int kPer = 8;                           // elements per thread and chunk: one 16-byte vector
constexpr int kChunkElems = kThreads * kPer;

struct SmallArParams {
  const float* parts;         // [slices][rows * cols] fp32
  int slices;
  int64_t slice_elems;
  int64_t total;              // rows * cols
  int64_t out_first, out_count;   // the elements this rank reduces and stores: all of them (all-reduce) or its rows (reduce-scatter)
  int cols;
  void* out;                  // local output: element out_first lands at out[0]; rows of `cols` elements, pitch ldc
  int64_t ldc;
  int fmt;                    // FMT_F16 / FMT_BF16
  int rank, W;
  uint8_t* part[8];           // every rank's buffer half of this epoch
  uint8_t* part_mc;           // multicast alias of it, or nullptr
  uint32_t* flags[8];         // every rank's stamp words [chunk][source]
  uint32_t* flags_mc;
  uint32_t* epoch_ptr;
  uint32_t* cta_counter;
  uint32_t* status;
  uint64_t timeout_ns;
};

__device__ __forceinline__ uint32_t pack2(float lo, float hi, int fmt) {
  if (fmt == FMT_BF16) { __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi); return *reinterpret_cast<uint32_t*>(&h); }
  __half2 h = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ void unpack2(uint32_t w, int fmt, float& lo, float& hi) {
  if (fmt == FMT_BF16) { const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w)); lo = f.x; hi = f.y; }
  else { const float2 f = __half22float2(*reinterpret_cast<__half2*>(&w)); lo = f.x; hi = f.y; }
}

__global__ void __launch_bounds__(kThreads) splitk_allreduce_kernel(const SmallArParams p) {
  __shared__ uint32_t s_fail[4];                  // [0] set, [1] source that did not arrive, [2] stamp seen, [3] chunk
  const int tid = threadIdx.x;
  if (*p.status != 0u) return;                    // an earlier failure is latched: do nothing, keep the epoch
  const uint32_t epoch = ptx::ld_relaxed_sys_u32(p.epoch_ptr) + 1u;
  const int64_t chunks = (p.total + kChunkElems - 1) / kChunkElems;
  if (tid == 0) s_fail[0] = 0u;
  __syncthreads();

  // ---- phase A: fold the K slices, publish this rank's copy ----
  for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    const int64_t e0 = c * kChunkElems + static_cast<int64_t>(tid) * kPer;
    if (e0 < p.total) {
      float acc[kPer] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int s = 0; s < p.slices; ++s) {
        const float4* src = reinterpret_cast<const float4*>(p.parts + s * p.slice_elems + e0);
        const float4 v0 = __ldg(src), v1 = __ldg(src + 1);
        acc[0] += v0.x; acc[1] += v0.y; acc[2] += v0.z; acc[3] += v0.w;
        acc[4] += v1.x; acc[5] += v1.y; acc[6] += v1.z; acc[7] += v1.w;
      }
      ptx::st_global_v4(p.part[p.rank] + e0 * 2, make_uint4(pack2(acc[0], acc[1], p.fmt), pack2(acc[2], acc[3], p.fmt),
                                                            pack2(acc[4], acc[5], p.fmt), pack2(acc[6], acc[7], p.fmt)));
    }
    __syncthreads();                              // the chunk's stores are ordered before the stamps below (cumulativity)
    if (p.flags_mc != nullptr) {
      if (tid == 0) { ptx::fence_acq_rel_sys(); ptx::multimem_st_release_u32(p.flags_mc + c * p.W + p.rank, epoch); }
    } else if (tid < p.W) {
      ptx::fence_acq_rel_sys();
      ptx::st_release_sys_u32(p.flags[tid] + c * p.W + p.rank, epoch);
    }
  }

  // ---- phase B: this rank sums the chunks of its output range (all of them for an all-reduce) ----
  bool failed = false;
  const int64_t c_lo = p.out_first / kChunkElems, c_hi = (p.out_first + p.out_count + kChunkElems - 1) / kChunkElems;
  for (int64_t c = c_lo + blockIdx.x; c < c_hi && !failed; c += gridDim.x) {
    if (tid < p.W) {
      const uint32_t* f = p.flags[p.rank] + c * p.W + tid;
      const uint64_t t0 = ptx::globaltimer_ns();
      uint32_t spins = 0;
      while (true) {
        const uint32_t v = ptx::ld_acquire_sys_u32(f);
        if (static_cast<int32_t>(v - epoch) >= 0) break;
        if ((++spins & 0xf) == 0) {
          if (ptx::globaltimer_ns() - t0 > p.timeout_ns || *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) {
            if (atomicCAS(&s_fail[0], 0u, 1u) == 0u) { s_fail[1] = tid; s_fail[2] = v; s_fail[3] = static_cast<uint32_t>(c); }
            break;
          }
          __nanosleep(64);
        }
      }
    }
    __syncthreads();
    if (s_fail[0] != 0u) { failed = true; break; }
    const int64_t e0 = c * kChunkElems + static_cast<int64_t>(tid) * kPer;
    if (e0 >= p.out_first && e0 < p.out_first + p.out_count) {
      uint4 r;
      if (p.part_mc != nullptr) {
        r = (p.fmt == FMT_BF16) ? ptx::multimem_ld_reduce_add_bf16x2_v4(p.part_mc + e0 * 2)
                                : ptx::multimem_ld_reduce_add_f16x2_v4(p.part_mc + e0 * 2);
      } else {
        float acc[kPer] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        for (int q = 0; q < p.W; ++q) {            // rank order: the same sum on every rank
          const uint4 v = ptx::ld_global_v4(p.part[q] + e0 * 2);
          const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) { float lo, hi; unpack2(w[j], p.fmt, lo, hi); acc[2 * j] += lo; acc[2 * j + 1] += hi; }
        }
        r = make_uint4(pack2(acc[0], acc[1], p.fmt), pack2(acc[2], acc[3], p.fmt), pack2(acc[4], acc[5], p.fmt),
                       pack2(acc[6], acc[7], p.fmt));
      }
      const int64_t eo = e0 - p.out_first;
      const int64_t row = eo / p.cols, col = eo - row * p.cols;     // cols % 8 == 0: a vector never crosses a row
      ptx::st_global_v4(static_cast<uint8_t*>(p.out) + (row * p.ldc + col) * 2, r);
    }
  }
  if (failed && tid == 0) {
    if (atomicCAS(p.status, 0u, static_cast<uint32_t>(STATUS_TIMEOUT_ARRIVE)) == 0u) {
      p.status[1] = epoch; p.status[2] = 300u; p.status[3] = epoch; p.status[4] = s_fail[2]; p.status[5] = s_fail[1];
      p.status[6] = blockIdx.x; p.status[7] = s_fail[3];
      __threadfence_system();
    }
  }

  // ---- the last CTA out advances the epoch ----
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.cta_counter = 0;
      __threadfence();
      if (*p.status == 0u) *p.epoch_ptr = epoch;
    }
  }
}


// ---------------------------------------------------------------------------------------------------------------
// All-gather of a small row-sharded activation, the first launch of the all-gather GEMM for few rows: every rank
// copies its shard [m, row_bytes] into rows [rank m, (rank + 1) m) of EVERY rank's gathered buffer (one multimem.st
// per 16 bytes, or a store per peer), stamps (chunk, rank) everywhere, then waits until the chunks of all W sources
// have landed in its own buffer. The split-K product that follows reads the gathered rows from local memory.
struct SmallAgParams {
  const uint8_t* shard;       // [m rows], pitch shard_pitch bytes, 16-byte aligned rows
  int64_t shard_pitch;
  int m;
  int64_t row_bytes;          // bytes copied per row (a multiple of 16)
  int64_t dst_pitch;          // pitch of the gathered buffer
  int rank, W;
  uint8_t* gathered[8];       // every rank's buffer half of this epoch
  uint8_t* gathered_mc;
  uint32_t* flags[8];         // stamp words [chunk][source]
  uint32_t* flags_mc;
  uint32_t* epoch_ptr;
  uint32_t* cta_counter;
  uint32_t* status;
  uint64_t timeout_ns;
};

__global__ void __launch_bounds__(kThreads) small_allgather_kernel(const SmallAgParams p) {
  __shared__ uint32_t s_fail[4];
  const int tid = threadIdx.x;
  if (*p.status != 0u) return;
  const uint32_t epoch = ptx::ld_relaxed_sys_u32(p.epoch_ptr) + 1u;
  const int64_t vec_per_row = p.row_bytes >> 4;
  const int64_t total = vec_per_row * p.m;                       // 16-byte vectors of the shard
  const int64_t chunks = (total + kThreads - 1) / kThreads;      // one vector per thread and chunk
  if (tid == 0) s_fail[0] = 0u;
  __syncthreads();

  // ---- phase A: send the shard ----
  for (int64_t c = blockIdx.x; c < chunks; c += gridDim.x) {
    const int64_t v = c * kThreads + tid;
    if (v < total) {
      const int64_t row = v / vec_per_row, u = v - row * vec_per_row;
      const uint4 x = ptx::ld_global_nc_v4(p.shard + row * p.shard_pitch + (u << 4));
      const int64_t off = (static_cast<int64_t>(p.rank) * p.m + row) * p.dst_pitch + (u << 4);
      if (p.gathered_mc != nullptr) ptx::multimem_st_v4(p.gathered_mc + off, x);
      else
        for (int q = 0; q < p.W; ++q) ptx::st_global_v4(p.gathered[q] + off, x);
    }
    __syncthreads();
    if (p.flags_mc != nullptr) {
      if (tid == 0) { ptx::fence_acq_rel_sys(); ptx::multimem_st_release_u32(p.flags_mc + c * p.W + p.rank, epoch); }
    } else if (tid < p.W) {
      ptx::fence_acq_rel_sys();
      ptx::st_release_sys_u32(p.flags[tid] + c * p.W + p.rank, epoch);
    }
  }

  // ---- phase B: wait for every source's chunks ----
  bool failed = false;
  for (int64_t c = blockIdx.x; c < chunks && !failed; c += gridDim.x) {
    if (tid < p.W) {
      const uint32_t* f = p.flags[p.rank] + c * p.W + tid;
      const uint64_t t0 = ptx::globaltimer_ns();
      uint32_t spins = 0;
      while (true) {
        const uint32_t v = ptx::ld_acquire_sys_u32(f);
        if (static_cast<int32_t>(v - epoch) >= 0) break;
        if ((++spins & 0xf) == 0) {
          if (ptx::globaltimer_ns() - t0 > p.timeout_ns || *reinterpret_cast<volatile uint32_t*>(p.status) != 0u) {
            if (atomicCAS(&s_fail[0], 0u, 1u) == 0u) { s_fail[1] = tid; s_fail[2] = v; s_fail[3] = static_cast<uint32_t>(c); }
            break;
          }
          __nanosleep(64);
        }
      }
    }
    __syncthreads();
    if (s_fail[0] != 0u) failed = true;
  }
  if (failed && tid == 0) {
    if (atomicCAS(p.status, 0u, static_cast<uint32_t>(STATUS_TIMEOUT_GATHER)) == 0u) {
      p.status[1] = epoch; p.status[2] = 301u; p.status[3] = epoch; p.status[4] = s_fail[2]; p.status[5] = s_fail[1];
      p.status[6] = blockIdx.x; p.status[7] = s_fail[3];
      __threadfence_system();
    }
  }
  __syncthreads();
  if (tid == 0) {
    __threadfence();
    const uint32_t prev = atomicAdd(p.cta_counter, 1u);
    if (prev == gridDim.x - 1) {
      *p.cta_counter = 0;
      __threadfence();
      if (*p.status == 0u) *p.epoch_ptr = epoch;
    }
  }
}

}  // namespace
}  // namespace catcoc

using namespace catcoc;

extern "C" int catcoc_splitk_allreduce(const CatcocShmemCtx* ctx, const float* parts, int slices, int64_t slice_elems,
                                       int rows, int cols, int out_row0, int out_rows, void* out, int64_t ldc, int fmt,
                                       int64_t part_off,
                                       int64_t flags_off, int use_multicast, uint32_t* epoch_ptr, uint32_t* cta_counter,
                                       uint32_t* status, uint64_t timeout_ns, void* stream) {
  if (ctx == nullptr || parts == nullptr || out == nullptr || epoch_ptr == nullptr || cta_counter == nullptr ||
      status == nullptr || slices <= 0 || rows <= 0 || cols <= 0 || ctx->W < 2 || ctx->W > 8 || out_row0 < 0 ||
      out_rows <= 0 || out_row0 + out_rows > rows) {
    host::set_error("splitk_allreduce: bad argument");
    return CATCOC_E_BAD_ARG;
  }
  if (fmt != CATCOC_FMT_F16 && fmt != CATCOC_FMT_BF16) { host::set_error("splitk_allreduce takes fp16 / bf16 outputs"); return CATCOC_E_UNSUPPORTED; }
  if ((cols % 8) != 0 || (ldc % 8) != 0 || (reinterpret_cast<uintptr_t>(out) & 15) != 0 || (part_off & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(parts) & 15) != 0 || (slice_elems % 4) != 0 || (flags_off & 3) != 0) {
    host::set_error("splitk_allreduce: rows of 8 elements and 16-byte aligned buffers are required");
    return CATCOC_E_ALIGNMENT;
  }
  SmallArParams p;
  p.parts = parts; p.slices = slices; p.slice_elems = slice_elems;
  p.total = static_cast<int64_t>(rows) * cols; p.cols = cols;
  p.out_first = static_cast<int64_t>(out_row0) * cols; p.out_count = static_cast<int64_t>(out_rows) * cols;
  p.out = out; p.ldc = ldc; p.fmt = fmt;
  p.rank = ctx->rank; p.W = ctx->W;
  for (int q = 0; q < 8; ++q) {
    p.part[q] = q < ctx->W ? static_cast<uint8_t*>(ctx->base[q]) + part_off : nullptr;
    p.flags[q] = q < ctx->W ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctx->base[q]) + flags_off) : nullptr;
  }
  const bool mc = use_multicast && ctx->mc_base != nullptr;
  p.part_mc = mc ? static_cast<uint8_t*>(ctx->mc_base) + part_off : nullptr;
  p.flags_mc = mc ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctx->mc_base) + flags_off) : nullptr;
  p.epoch_ptr = epoch_ptr; p.cta_counter = cta_counter; p.status = status;
  p.timeout_ns = timeout_ns ? timeout_ns : 10000000000ull;
  const int64_t chunks = (p.total + kChunkElems - 1) / kChunkElems;
  const int grid = static_cast<int>(chunks < 148 * 4 ? chunks : 148 * 4);
  splitk_allreduce_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int64_t catcoc_splitk_allreduce_flag_words(int rows, int cols, int W) {
  const int64_t total = static_cast<int64_t>(rows) * cols;
  return (total + kChunkElems - 1) / kChunkElems * W;
}

extern "C" int64_t catcoc_small_allgather_flag_words(int m, int64_t row_bytes, int W) {
  const int64_t total = (row_bytes >> 4) * m;
  return (total + kThreads - 1) / kThreads * W;
}

extern "C" int catcoc_small_allgather(const CatcocShmemCtx* ctx, const void* shard, int64_t shard_pitch_bytes, int m,
                                      int64_t row_bytes, int64_t gathered_off, int64_t gathered_pitch_bytes,
                                      int64_t flags_off, int use_multicast, uint32_t* epoch_ptr, uint32_t* cta_counter,
                                      uint32_t* status, uint64_t timeout_ns, void* stream) {
  if (ctx == nullptr || shard == nullptr || epoch_ptr == nullptr || cta_counter == nullptr || status == nullptr || m <= 0 ||
      row_bytes <= 0 || ctx->W < 2 || ctx->W > 8) {
    host::set_error("small_allgather: bad argument");
    return CATCOC_E_BAD_ARG;
  }
  if ((row_bytes & 15) != 0 || (shard_pitch_bytes & 15) != 0 || (gathered_pitch_bytes & 15) != 0 || (gathered_off & 15) != 0 ||
      (reinterpret_cast<uintptr_t>(shard) & 15) != 0 || (flags_off & 3) != 0 || gathered_pitch_bytes < row_bytes ||
      shard_pitch_bytes < row_bytes) {
    host::set_error("small_allgather: rows of whole 16-byte vectors and 16-byte aligned buffers are required");
    return CATCOC_E_ALIGNMENT;
  }
  SmallAgParams p;
  p.shard = static_cast<const uint8_t*>(shard); p.shard_pitch = shard_pitch_bytes; p.m = m; p.row_bytes = row_bytes;
  p.dst_pitch = gathered_pitch_bytes;
  p.rank = ctx->rank; p.W = ctx->W;
  for (int q = 0; q < 8; ++q) {
    p.gathered[q] = q < ctx->W ? static_cast<uint8_t*>(ctx->base[q]) + gathered_off : nullptr;
    p.flags[q] = q < ctx->W ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctx->base[q]) + flags_off) : nullptr;
  }
  const bool mc = use_multicast && ctx->mc_base != nullptr;
  p.gathered_mc = mc ? static_cast<uint8_t*>(ctx->mc_base) + gathered_off : nullptr;
  p.flags_mc = mc ? reinterpret_cast<uint32_t*>(static_cast<uint8_t*>(ctx->mc_base) + flags_off) : nullptr;
  p.epoch_ptr = epoch_ptr; p.cta_counter = cta_counter; p.status = status;
  p.timeout_ns = timeout_ns ? timeout_ns : 10000000000ull;
  const int64_t chunks = ((row_bytes >> 4) * m + kThreads - 1) / kThreads;
  const int grid = static_cast<int>(chunks < 148 * 4 ? chunks : 148 * 4);
  small_allgather_kernel<<<grid, kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}
