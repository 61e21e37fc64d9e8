// Allocation-free variant of the padded-operand GEMM path; see catcoc/no_alloc.h for who needs
// it and the rules of use. Nothing in this file (or in what it calls) allocates device memory.
#include <cstring>
#include "catcoc/capi.h"
#include "catcoc/fused_gemm.cuh"
#include "catcoc/host_util.h"
#include "catcoc/no_alloc.h"

using namespace catcoc;
using namespace catcoc::host;

// Implemented in launch.cu / shmem_prims.cu.
int catcoc_build_params(const CatcocOpArgs* args, FusedParams* p, int* kind_out, int* grid_out, int* pair_out);
int catcoc_launch_params(const FusedParams& p, int kind, int grid, int pair, int threads, cudaStream_t stream);

// The scratch area. In host code this name is only a stand-in for the symbol: it is NOT a
// device address and must never be handed to a kernel or a copy. Host code uses the address
// that cudaGetSymbolAddress returns for the current device (resolve_scratch below).
// Layout: [0, 256) status words | padded A | padded B.
static __device__ __align__(256) unsigned char g_noalloc_scratch[CATCOC_NOALLOC_SCRATCH_BYTES];

namespace {

constexpr int kMaxDevices = 64;
// Per device, filled on first use. Two host threads that make their first call on the same device at
// the same time both resolve the symbol and store the same address: the race is benign (an aligned
// pointer store of one value), so the table carries no lock.
unsigned char* g_scratch_addr[kMaxDevices];

// Once per device, with that device current.
int resolve_scratch(unsigned char** out) {
  int device = -1;
  CATCOC_CUDA_OK(cudaGetDevice(&device));
  if (device < 0 || device >= kMaxDevices) {
    set_error("device index %d out of range", device);
    return CATCOC_E_BAD_ARG;
  }
  if (g_scratch_addr[device] == nullptr) {
    void* ptr = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&ptr, g_noalloc_scratch);
    if (e != cudaSuccess || ptr == nullptr) {
      set_error("cudaGetSymbolAddress(scratch) failed on device %d: %s", device, cudaGetErrorString(e));
      return -1000 - static_cast<int>(e);
    }
    g_scratch_addr[device] = static_cast<unsigned char*>(ptr);
  }
  *out = g_scratch_addr[device];
  return CATCOC_OK;
}

// Copies rows into a buffer with a 16-byte-multiple pitch and zero-fills the padding, so no
// byte of the destination keeps what an earlier call left there.
// Destination rows are 16-byte aligned (pitch a multiple of 16, base 256-byte aligned); a source row
// that is 16- or 4-byte aligned is moved in units of that size, the ragged end and rows of any other
// alignment byte by byte.
__global__ void noalloc_pad_kernel(unsigned char* dst, long long dst_pitch, const unsigned char* src,
                                   long long src_pitch, long long rows, long long row_bytes) {
  for (long long r = blockIdx.x; r < rows; r += gridDim.x) {
    const unsigned char* s = src + r * src_pitch;
    unsigned char* d = dst + r * dst_pitch;
    const unsigned long long sa = reinterpret_cast<unsigned long long>(s);
    long long done = 0;
    if ((sa & 15ull) == 0) {
      const long long n16 = row_bytes >> 4;
      for (long long i = threadIdx.x; i < n16; i += blockDim.x)
        reinterpret_cast<uint4*>(d)[i] = reinterpret_cast<const uint4*>(s)[i];
      done = n16 << 4;
    } else if ((sa & 3ull) == 0) {
      const long long n4 = row_bytes >> 2;
      for (long long i = threadIdx.x; i < n4; i += blockDim.x)
        reinterpret_cast<unsigned int*>(d)[i] = reinterpret_cast<const unsigned int*>(s)[i];
      done = n4 << 2;
    }
    for (long long b = done + threadIdx.x; b < dst_pitch; b += blockDim.x)
      d[b] = (b < row_bytes) ? s[b] : static_cast<unsigned char>(0);
  }
}

int elt_bytes_of(int in_fmt) {
  switch (in_fmt) {
    case CATCOC_IN_F16: case CATCOC_IN_BF16: return 2;
    case CATCOC_IN_S8: case CATCOC_IN_E4M3: case CATCOC_IN_E5M2: return 1;
    default: return 0;
  }
}

}  // namespace

extern "C" int catcoc_matmul_noalloc(const void* a, int64_t lda, const void* b, int64_t ldb, void* out, int64_t ldc,
                                     int M, int N, int K, int in_fmt, int out_fmt, int trans_a, int trans_b,
                                     void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  const int elt = elt_bytes_of(in_fmt);
  if (a == nullptr || b == nullptr || out == nullptr || M <= 0 || N <= 0 || K <= 0 || elt == 0) {
    set_error("matmul_noalloc: bad arguments");
    return CATCOC_E_BAD_ARG;
  }
  // stored shapes (rows x cols, cols contiguous)
  const int64_t a_rows = trans_a ? K : M, a_cols = trans_a ? M : K;
  const int64_t b_rows = trans_b ? N : K, b_cols = trans_b ? K : N;
  if (lda < a_cols || ldb < b_cols || ldc < N) {
    set_error("matmul_noalloc: leading dimension smaller than the row length");
    return CATCOC_E_BAD_ARG;
  }
  const int per16 = 16 / elt;
  const int64_t a_ld = (a_cols + per16 - 1) / per16 * per16;
  const int64_t b_ld = (b_cols + per16 - 1) / per16 * per16;
  const int64_t a_bytes = a_rows * a_ld * elt, b_bytes = b_rows * b_ld * elt;
  if (a_bytes > static_cast<int64_t>(CATCOC_NOALLOC_OPERAND_BYTES) ||
      b_bytes > static_cast<int64_t>(CATCOC_NOALLOC_OPERAND_BYTES)) {
    set_error("matmul_noalloc: padded operands need %lld and %lld bytes, the built-in scratch holds %u bytes per "
              "operand; use the regular entry point for larger problems",
              static_cast<long long>(a_bytes), static_cast<long long>(b_bytes), CATCOC_NOALLOC_OPERAND_BYTES);
    return CATCOC_E_TOO_LARGE;
  }
  unsigned char* scratch = nullptr;
  int rc = resolve_scratch(&scratch);
  if (rc != 0) return rc;
  uint32_t* status = reinterpret_cast<uint32_t*>(scratch);
  unsigned char* a_pad = scratch + 256;
  unsigned char* b_pad = a_pad + CATCOC_NOALLOC_OPERAND_BYTES;

  // the status words must start at zero; the operand areas are fully rewritten below
  CATCOC_CUDA_OK(cudaMemsetAsync(status, 0, 256, stream));
  const int ga = a_rows < 1184 ? static_cast<int>(a_rows) : 1184;
  const int gb = b_rows < 1184 ? static_cast<int>(b_rows) : 1184;
  noalloc_pad_kernel<<<ga, 256, 0, stream>>>(a_pad, a_ld * elt, static_cast<const unsigned char*>(a), lda * elt, a_rows,
                                             a_cols * elt);
  noalloc_pad_kernel<<<gb, 256, 0, stream>>>(b_pad, b_ld * elt, static_cast<const unsigned char*>(b), ldb * elt, b_rows,
                                             b_cols * elt);
  CATCOC_CUDA_OK(cudaGetLastError());

  CatcocOpArgs args;
  memset(&args, 0, sizeof(args));
  args.mode = CATCOC_MODE_LOCAL;
  args.in_fmt = in_fmt;
  args.M = M; args.N = N; args.K = K;
  args.trans_a = trans_a; args.trans_b = trans_b;
  args.a = a_pad; args.lda = a_ld;
  args.b = b_pad; args.ldb = b_ld;
  args.out = out; args.ldc = ldc; args.out_fmt = out_fmt;
  args.partial_fmt = out_fmt;
  args.rank = 0; args.W = 1;
  args.status = status;
  FusedParams p;
  int kind = 0, grid = 0, pair = 0;
  rc = catcoc_build_params(&args, &p, &kind, &grid, &pair);
  if (rc != 0) return rc;
  return catcoc_launch_params(p, kind, grid, pair, 0, stream);
}

extern "C" int catcoc_matmul_noalloc_status(uint32_t* host_words) {
  if (host_words == nullptr) return CATCOC_E_BAD_ARG;
  unsigned char* scratch = nullptr;
  int rc = resolve_scratch(&scratch);
  if (rc != 0) return rc;
  CATCOC_CUDA_OK(cudaMemcpy(host_words, scratch, 8 * sizeof(uint32_t), cudaMemcpyDeviceToHost));
  return CATCOC_OK;
}
