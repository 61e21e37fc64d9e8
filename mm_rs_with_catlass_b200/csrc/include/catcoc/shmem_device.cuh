// Device-side SHMEM API over the symmetric heap: address translation, cooperative put / get,
// signals, bounded waits and a device-callable barrier across all ranks.
//
// Counterpart of the SHMEM device calls the reference uses (shmem_my_pe / shmem_n_pes /
// shmem_mte_put_mem_nbi / shmem_mte_get_mem_nbi / shmemx_barrier_all_vec,
// include/catcoc/comm_epilogue/tile/tile_remote_copy.hpp:63-102 and
// include/catcoc/dgemm/kernel/matmul_allreduce.hpp:251-309) plus put_signal / wait_until,
// which the reference does not have. Data moves with plain 16-byte loads and stores on
// peer-mapped addresses (NVLink P2P) or multimem instructions on the multicast alias.
// Every wait is bounded and returns false on time-out.
#pragma once
#include "catcoc/ptx.cuh"

namespace catcoc {
namespace shmem {

struct Ctx {
  int rank, W;
  uint8_t* base[8];   // heap base of every rank, as mapped in this process
  uint8_t* mc_base;   // multicast alias of the heap, or nullptr
};

CATCOC_DEVICE int my_pe(const Ctx& c) { return c.rank; }
CATCOC_DEVICE int n_pes(const Ctx& c) { return c.W; }

// Address of the symmetric object at byte offset `off` on rank `pe`.
template <typename T = uint8_t>
CATCOC_DEVICE T* ptr(const Ctx& c, int64_t off, int pe) {
  return reinterpret_cast<T*>(c.base[pe] + off);
}
template <typename T = uint8_t>
CATCOC_DEVICE T* mc_ptr(const Ctx& c, int64_t off) {
  return c.mc_base ? reinterpret_cast<T*>(c.mc_base + off) : nullptr;
}

// Orders this thread's earlier stores before its later ones at system scope (fence) and is
// also what "quiet" reduces to for plain stores: they are posted, and the release on the
// following signal makes them visible before it.
CATCOC_DEVICE void fence() { ptx::fence_acq_rel_sys(); }
CATCOC_DEVICE void quiet() { ptx::fence_acq_rel_sys(); }

// Cooperative copy of `bytes` (16-byte aligned both sides, multiple of 16) by `nthreads`
// threads with index `tid`; tail bytes are copied by thread 0.
CATCOC_DEVICE void copy_coop(uint8_t* dst, const uint8_t* src, int64_t bytes, int tid, int nthreads) {
  const int64_t n16 = bytes >> 4;
  int64_t i = tid;
  for (; i + 3 * nthreads < n16; i += 4 * nthreads) {
    uint4 v0 = ptx::ld_global_v4(src + (i << 4));
    uint4 v1 = ptx::ld_global_v4(src + ((i + nthreads) << 4));
    uint4 v2 = ptx::ld_global_v4(src + ((i + 2 * nthreads) << 4));
    uint4 v3 = ptx::ld_global_v4(src + ((i + 3 * nthreads) << 4));
    ptx::st_global_v4(dst + (i << 4), v0);
    ptx::st_global_v4(dst + ((i + nthreads) << 4), v1);
    ptx::st_global_v4(dst + ((i + 2 * nthreads) << 4), v2);
    ptx::st_global_v4(dst + ((i + 3 * nthreads) << 4), v3);
  }
  for (; i < n16; i += nthreads) ptx::st_global_v4(dst + (i << 4), ptx::ld_global_v4(src + (i << 4)));
  if (tid == 0)
    for (int64_t b = n16 << 4; b < bytes; ++b) dst[b] = src[b];
}

// put: local `src` -> symmetric offset `dst_off` on rank `pe`. Non-blocking in the SHMEM
// sense: completion is only guaranteed after quiet()/a signal.
CATCOC_DEVICE void put(const Ctx& c, int pe, int64_t dst_off, const void* src, int64_t bytes, int tid, int nthreads) {
  copy_coop(ptr(c, dst_off, pe), static_cast<const uint8_t*>(src), bytes, tid, nthreads);
}
// get: symmetric offset `src_off` on rank `pe` -> local `dst`.
CATCOC_DEVICE void get(const Ctx& c, int pe, void* dst, int64_t src_off, int64_t bytes, int tid, int nthreads) {
  copy_coop(static_cast<uint8_t*>(dst), ptr(c, src_off, pe), bytes, tid, nthreads);
}

// 2-D strided variants (rows x row_bytes with independent pitches), the shape of the
// reference's non_contiguous_copy_param{repeat, length, src_ld, dst_ld}.
CATCOC_DEVICE void put_2d(const Ctx& c, int pe, int64_t dst_off, int64_t dst_pitch, const void* src,
                          int64_t src_pitch, int rows, int64_t row_bytes, int tid, int nthreads) {
  const int64_t per_row = row_bytes >> 4;
  const int64_t total = per_row * rows;
  uint8_t* d = ptr(c, dst_off, pe);
  const uint8_t* s = static_cast<const uint8_t*>(src);
  for (int64_t i = tid; i < total; i += nthreads) {
    const int64_t r = i / per_row, u = i - r * per_row;
    ptx::st_global_v4(d + r * dst_pitch + (u << 4), ptx::ld_global_v4(s + r * src_pitch + (u << 4)));
  }
}

enum SignalOp { SIGNAL_SET = 0, SIGNAL_ADD = 1 };

// One thread: make this thread's (and, after a CTA/warp barrier, its group's) earlier stores
// visible system-wide, then update the 32-bit signal word on rank `pe`.
CATCOC_DEVICE void signal_op(const Ctx& c, int pe, int64_t sig_off, uint32_t value, int op) {
  uint32_t* s = ptr<uint32_t>(c, sig_off, pe);
  ptx::fence_acq_rel_sys();
  if (op == SIGNAL_SET) ptx::st_release_sys_u32(s, value);
  else ptx::red_release_sys_add_u32(s, value);
}

// put + signal from one CTA: every thread copies, all fence, then thread 0 signals.
CATCOC_DEVICE void put_signal_block(const Ctx& c, int pe, int64_t dst_off, const void* src, int64_t bytes,
                                    int64_t sig_off, uint32_t value, int op) {
  put(c, pe, dst_off, src, bytes, threadIdx.x, blockDim.x);
  ptx::fence_acq_rel_sys();
  __syncthreads();
  if (threadIdx.x == 0) signal_op(c, pe, sig_off, value, op);
}

// Bounded wait until the local signal word is >= value (wrap-safe). Returns false on time-out.
CATCOC_DEVICE bool wait_until_ge(const Ctx& c, int64_t sig_off, uint32_t value, uint64_t timeout_ns, uint32_t* seen) {
  const uint32_t* s = ptr<uint32_t>(c, sig_off, c.rank);
  const uint64_t t0 = ptx::globaltimer_ns();
  uint32_t spins = 0;
  while (true) {
    const uint32_t v = ptx::ld_acquire_sys_u32(s);
    if (static_cast<int32_t>(v - value) >= 0) return true;
    if ((++spins & 0xf) == 0) {
      if (ptx::globaltimer_ns() - t0 > timeout_ns) {
        if (seen) *seen = v;
        return false;
      }
      __nanosleep(100);
    }
  }
}

// Barrier across all ranks, callable by one CTA in the middle of a kernel. `bar_off` names W
// 32-bit words in the heap; `epoch` must grow by one per barrier on every rank (stamps are
// never reset, so back-to-back barriers and graph replays need no clean-up).
// Returns false if a peer did not arrive in time.
CATCOC_DEVICE bool barrier_all_block(const Ctx& c, int64_t bar_off, uint32_t epoch, uint64_t timeout_ns, uint32_t* seen_peer) {
  ptx::fence_acq_rel_sys();
  __syncthreads();
  __shared__ int s_ok;
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (static_cast<int>(threadIdx.x) < c.W) {
    const int pe = threadIdx.x;
    ptx::st_release_sys_u32(ptr<uint32_t>(c, bar_off, pe) + c.rank, epoch);
    uint32_t seen = 0;
    if (!wait_until_ge(c, bar_off + 4 * pe, epoch, timeout_ns, &seen)) {
      s_ok = 0;
      if (seen_peer) *seen_peer = static_cast<uint32_t>(pe);
    }
  }
  __syncthreads();
  return s_ok != 0;
}

}  // namespace shmem
}  // namespace catcoc
