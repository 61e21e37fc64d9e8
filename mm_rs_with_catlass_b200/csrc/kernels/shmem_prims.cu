// Stand-alone kernels around the device SHMEM API: barrier_all, put (+signal), get, wait_until,
// NVLS broadcast and NVLS reduce. They back the Python-level `SymmetricHeap.barrier()` and the
// primitive tests; the fused ops inline the same device functions instead of launching these.
#include "catcoc/capi.h"
#include "catcoc/host_util.h"
#include "catcoc/params.h"
#include "catcoc/shmem_device.cuh"

using namespace catcoc;

namespace {

shmem::Ctx to_ctx(const CatcocShmemCtx* c) {
  shmem::Ctx d;
  d.rank = c->rank;
  d.W = c->W;
  for (int i = 0; i < 8; ++i) d.base[i] = static_cast<uint8_t*>(c->base[i]);
  d.mc_base = static_cast<uint8_t*>(c->mc_base);
  return d;
}

__device__ void set_status(uint32_t* status, uint32_t code, uint32_t rank, uint32_t what, uint32_t expected,
                           uint32_t seen, uint32_t peer) {
  if (status == nullptr) return;
  if (atomicCAS(status, 0u, code) == 0u) {
    status[1] = rank; status[2] = what; status[3] = expected; status[4] = seen; status[5] = peer;
    status[6] = blockIdx.x;
  }
}

__global__ void barrier_all_kernel(shmem::Ctx c, int64_t bar_off, uint32_t epoch, uint64_t timeout_ns, uint32_t* status) {
  uint32_t peer = 0;
  if (!shmem::barrier_all_block(c, bar_off, epoch, timeout_ns, &peer) && threadIdx.x == 0)
    set_status(status, STATUS_TIMEOUT_BARRIER, c.rank, 0u, epoch, 0u, peer);
}

__global__ void put_kernel(shmem::Ctx c, int peer, int64_t dst_off, const uint8_t* src, int64_t bytes,
                           int64_t sig_off, uint32_t sig_val) {
  // grid-stride over 16-byte units; the last block to finish posts the signal
  const int64_t chunk = (bytes + gridDim.x - 1) / gridDim.x;
  const int64_t begin = ((static_cast<int64_t>(blockIdx.x) * chunk) + 15) & ~int64_t(15);
  int64_t end = ((static_cast<int64_t>(blockIdx.x + 1) * chunk) + 15) & ~int64_t(15);
  if (end > bytes) end = bytes;
  if (begin < end) shmem::put(c, peer, dst_off + begin, src + begin, end - begin, threadIdx.x, blockDim.x);
  if (sig_off >= 0) {
    ptx::fence_acq_rel_sys();
    __syncthreads();
    // every block adds 1; the receiver waits for value * gridDim.x via the host-side wrapper
    if (threadIdx.x == 0) shmem::signal_op(c, peer, sig_off, sig_val, shmem::SIGNAL_ADD);
  }
}

__global__ void get_kernel(shmem::Ctx c, int peer, uint8_t* dst, int64_t src_off, int64_t bytes) {
  const int64_t chunk = (bytes + gridDim.x - 1) / gridDim.x;
  const int64_t begin = ((static_cast<int64_t>(blockIdx.x) * chunk) + 15) & ~int64_t(15);
  int64_t end = ((static_cast<int64_t>(blockIdx.x + 1) * chunk) + 15) & ~int64_t(15);
  if (end > bytes) end = bytes;
  if (begin < end) shmem::get(c, peer, dst + begin, src_off + begin, end - begin, threadIdx.x, blockDim.x);
}

__global__ void wait_until_kernel(shmem::Ctx c, int64_t sig_off, uint32_t value, uint64_t timeout_ns, uint32_t* status) {
  uint32_t seen = 0;
  if (threadIdx.x == 0 && !shmem::wait_until_ge(c, sig_off, value, timeout_ns, &seen))
    set_status(status, STATUS_TIMEOUT_BARRIER, c.rank, 1u, value, seen, 0u);
}

__global__ void mc_broadcast_kernel(shmem::Ctx c, int64_t dst_off, const uint8_t* src, int64_t bytes) {
  uint8_t* mc = shmem::mc_ptr(c, dst_off);
  const int64_t n16 = bytes >> 4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    ptx::multimem_st_v4(mc + (i << 4), ptx::ld_global_v4(src + (i << 4)));
}

__global__ void mc_reduce_bf16_kernel(shmem::Ctx c, uint8_t* dst, int64_t src_off, int64_t n_elems) {
  const uint8_t* mc = shmem::mc_ptr(c, src_off);
  const int64_t n16 = (n_elems * 2) >> 4;
  for (int64_t i = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; i < n16;
       i += static_cast<int64_t>(gridDim.x) * blockDim.x)
    ptx::st_global_v4(dst + (i << 4), ptx::multimem_ld_reduce_add_bf16x2_v4(mc + (i << 4)));
}

// 2-D copy with independent pitches and zero fill of the padding columns: makes a TMA-legal
// (16-byte pitch) copy of a matrix whose leading dimension is not.
__global__ void pad2d_kernel(uint8_t* dst, int64_t dst_pitch, const uint8_t* src, int64_t src_pitch, int64_t rows,
                             int64_t row_bytes) {
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint8_t* s = src + r * src_pitch;
    uint8_t* d = dst + r * dst_pitch;
    for (int64_t b = threadIdx.x; b < dst_pitch; b += blockDim.x) d[b] = (b < row_bytes) ? s[b] : uint8_t(0);
  }
}

}  // namespace

extern "C" int catcoc_shmem_barrier_all(const CatcocShmemCtx* ctx, uint32_t epoch, uint64_t timeout_ns,
                                        uint32_t* status, void* stream) {
  if (ctx == nullptr) return CATCOC_E_BAD_ARG;
  barrier_all_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), ctx->barrier_off, epoch,
                                                                      timeout_ns ? timeout_ns : 10000000000ull, status);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

// The signal word (if sig_off >= 0) receives `signal_val` once per launched block; this
// wrapper launches a fixed number of blocks and reports it so the receiver knows what to expect.
static const int kPutBlocks = 32;
extern "C" int catcoc_shmem_put_blocks(void) { return kPutBlocks; }

extern "C" int catcoc_shmem_put(const CatcocShmemCtx* ctx, int peer, int64_t dst_off, const void* src, int64_t bytes,
                                int64_t signal_off, uint32_t signal_val, void* stream) {
  if (ctx == nullptr || peer < 0 || peer >= ctx->W || (dst_off & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) {
    host::set_error("shmem_put: bad peer or unaligned addresses");
    return CATCOC_E_BAD_ARG;
  }
  put_kernel<<<kPutBlocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), peer, dst_off,
                                                                        static_cast<const uint8_t*>(src), bytes,
                                                                        signal_off, signal_val);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int catcoc_shmem_get(const CatcocShmemCtx* ctx, int peer, void* dst, int64_t src_off, int64_t bytes,
                                void* stream) {
  if (ctx == nullptr || peer < 0 || peer >= ctx->W || (src_off & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) {
    host::set_error("shmem_get: bad peer or unaligned addresses");
    return CATCOC_E_BAD_ARG;
  }
  get_kernel<<<kPutBlocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), peer, static_cast<uint8_t*>(dst),
                                                                        src_off, bytes);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int catcoc_shmem_wait_until(const CatcocShmemCtx* ctx, int64_t signal_off, uint32_t value,
                                       uint64_t timeout_ns, uint32_t* status, void* stream) {
  if (ctx == nullptr) return CATCOC_E_BAD_ARG;
  wait_until_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), signal_off, value,
                                                                     timeout_ns ? timeout_ns : 10000000000ull, status);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int catcoc_shmem_mc_broadcast(const CatcocShmemCtx* ctx, int64_t dst_off, const void* src, int64_t bytes,
                                         void* stream) {
  if (ctx == nullptr || ctx->mc_base == nullptr) { host::set_error("no multicast mapping"); return CATCOC_E_UNSUPPORTED; }
  if ((dst_off & 15) || (bytes & 15) || (reinterpret_cast<uintptr_t>(src) & 15)) { host::set_error("mc_broadcast: 16-byte alignment required"); return CATCOC_E_ALIGNMENT; }
  mc_broadcast_kernel<<<64, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), dst_off,
                                                                         static_cast<const uint8_t*>(src), bytes);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int catcoc_shmem_mc_reduce_bf16(const CatcocShmemCtx* ctx, void* dst, int64_t src_off, int64_t n_elems,
                                           void* stream) {
  if (ctx == nullptr || ctx->mc_base == nullptr) { host::set_error("no multicast mapping"); return CATCOC_E_UNSUPPORTED; }
  if ((src_off & 15) || (n_elems & 7) || (reinterpret_cast<uintptr_t>(dst) & 15)) { host::set_error("mc_reduce: 16-byte alignment required"); return CATCOC_E_ALIGNMENT; }
  mc_reduce_bf16_kernel<<<64, 256, 0, static_cast<cudaStream_t>(stream)>>>(to_ctx(ctx), static_cast<uint8_t*>(dst),
                                                                           src_off, n_elems);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int catcoc_pad2d(void* dst, int64_t dst_pitch, const void* src, int64_t src_pitch, int64_t rows,
                            int64_t row_bytes, void* stream) {
  if (rows <= 0) return CATCOC_OK;
  const int grid = rows < 1184 ? static_cast<int>(rows) : 1184;
  pad2d_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<uint8_t*>(dst), dst_pitch,
                                                                    static_cast<const uint8_t*>(src), src_pitch, rows,
                                                                    row_bytes);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}
