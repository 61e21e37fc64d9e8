// Bandwidth-bound companions of the tensor-core kernel: the reduction that finishes a split-K
// product and the matrix-vector products. Neither has a contraction large enough for tcgen05:
// both stream their operand once from HBM with 16-byte loads and accumulate in fp32.
//
// Counterparts in the reference's GEMM template library: the ReduceAdd stage of
// 3rdparty/catlass/include/catlass/gemm/kernel/splitk_matmul.hpp:30-160 and the vector-core GEMV
// 3rdparty/catlass/include/catlass/gemv/kernel/kernel_gemv_aiv.hpp (z = alpha * A x + beta * y).
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "catcoc/capi.h"
#include "catcoc/host_util.h"
#include "catcoc/params.h"

using namespace catcoc;

namespace {

__device__ __forceinline__ float load_elem(const void* p, int64_t i, int fmt) {
  if (fmt == FMT_F32) return static_cast<const float*>(p)[i];
  if (fmt == FMT_BF16) return __bfloat162float(static_cast<const __nv_bfloat16*>(p)[i]);
  return __half2float(static_cast<const __half*>(p)[i]);
}

__device__ __forceinline__ void store_elem(void* p, int64_t i, int fmt, float v) {
  if (fmt == FMT_F32) static_cast<float*>(p)[i] = v;
  else if (fmt == FMT_BF16) static_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else static_cast<__half*>(p)[i] = __float2half_rn(v);
}

__device__ __forceinline__ uint4 ldg_v4(const void* p) { return __ldg(static_cast<const uint4*>(p)); }

// Eight (16-bit formats) or four (fp32) consecutive elements of a 16-byte word as floats.
__device__ __forceinline__ int unpack_word(const uint4& w, int fmt, float* f) {
  const uint32_t u[4] = {w.x, w.y, w.z, w.w};
  if (fmt == FMT_F32) {
#pragma unroll
    for (int i = 0; i < 4; ++i) f[i] = __uint_as_float(u[i]);
    return 4;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (fmt == FMT_BF16) {
      f[2 * i] = __uint_as_float(u[i] << 16);
      f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    } else {
      const __half2 h = *reinterpret_cast<const __half2*>(&u[i]);
      f[2 * i] = __low2float(h);
      f[2 * i + 1] = __high2float(h);
    }
  }
  return 8;
}

// out[r, c] = cast(alpha * sum_s parts[s, r, c] + beta * c_src[r, c] + bias[c]); parts fp32
// [slices, rows, cols] with row pitch `cols`. One thread per 4 columns when cols % 4 == 0.
__global__ void splitk_reduce_kernel(const float* __restrict__ parts, int slices, int64_t slice_elems, int rows,
                                     int cols, void* out, int64_t ldc, int out_fmt, float alpha, float beta,
                                     const void* c_src, int64_t ldc_src, const float* __restrict__ bias) {
  const bool vec = (cols % 4) == 0;
  const int per = vec ? 4 : 1;
  const int64_t units = static_cast<int64_t>(rows) * (cols / per);
  for (int64_t u = blockIdx.x * static_cast<int64_t>(blockDim.x) + threadIdx.x; u < units;
       u += static_cast<int64_t>(gridDim.x) * blockDim.x) {
    const int r = static_cast<int>(u / (cols / per));
    const int c0 = static_cast<int>(u % (cols / per)) * per;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const int64_t off = static_cast<int64_t>(r) * cols + c0;
    for (int s = 0; s < slices; ++s) {
      const float* src = parts + s * slice_elems + off;
      if (vec) {
        const float4 v = __ldg(reinterpret_cast<const float4*>(src));
        acc[0] += v.x; acc[1] += v.y; acc[2] += v.z; acc[3] += v.w;
      } else {
        acc[0] += __ldg(src);
      }
    }
    for (int j = 0; j < per; ++j) {
      float v = alpha * acc[j];
      if (c_src != nullptr) v += beta * load_elem(c_src, static_cast<int64_t>(r) * ldc_src + c0 + j, out_fmt);
      if (bias != nullptr) v += __ldg(bias + c0 + j);
      store_elem(out, static_cast<int64_t>(r) * ldc + c0 + j, out_fmt, v);
    }
  }
}

// y[r] = alpha * sum_c A[r, c] * x[c] + beta * y_in[r]; A row-major with pitch lda. One group of
// TPR threads (a warp, or the whole 256-thread block for few long rows) per row.
template <int TPR>
__global__ void gemv_rows_kernel(const void* __restrict__ A, int64_t lda, int fmt, int rows, int cols,
                                 const void* __restrict__ x, void* y, const void* y_in, float alpha, float beta) {
  __shared__ float red[8];
  const int groups_per_block = blockDim.x / TPR;
  const int g = threadIdx.x / TPR;
  const int t = threadIdx.x % TPR;
  const int elt = (fmt == FMT_F32) ? 4 : 2;
  const int per = 16 / elt;
  for (int r = blockIdx.x * groups_per_block + g; r < rows; r += gridDim.x * groups_per_block) {
    const uint8_t* row = static_cast<const uint8_t*>(A) + static_cast<int64_t>(r) * lda * elt;
    const bool vec = ((reinterpret_cast<uintptr_t>(row) | reinterpret_cast<uintptr_t>(x)) & 15) == 0;
    float acc = 0.f;
    int c = 0;
    if (vec) {
      const int nvec = cols / per;
      int v = t;
      // four independent 16-byte loads of A in flight per thread (x comes from L1 / L2)
      for (; v + 3 * TPR < nvec; v += 4 * TPR) {
        uint4 wa[4], wx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          wa[j] = ldg_v4(row + static_cast<int64_t>(v + j * TPR) * 16);
          wx[j] = ldg_v4(static_cast<const uint8_t*>(x) + static_cast<int64_t>(v + j * TPR) * 16);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float fa[8], fx[8];
          unpack_word(wa[j], fmt, fa);
          unpack_word(wx[j], fmt, fx);
#pragma unroll
          for (int i = 0; i < 8; ++i)
            if (i < per) acc += fa[i] * fx[i];
        }
      }
      for (; v < nvec; v += TPR) {
        float fa[8], fx[8];
        unpack_word(ldg_v4(row + static_cast<int64_t>(v) * 16), fmt, fa);
        unpack_word(ldg_v4(static_cast<const uint8_t*>(x) + static_cast<int64_t>(v) * 16), fmt, fx);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < per) acc += fa[i] * fx[i];
      }
      c = nvec * per;
    }
    for (int i = c + t; i < cols; i += TPR) acc += load_elem(row, i, fmt) * load_elem(x, i, fmt);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    if (TPR > 32) {
      // the block works on one row: fold the warps' sums through shared memory
      __syncthreads();
      if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
      __syncthreads();
      acc = 0.f;
      for (int w = 0; w < TPR / 32; ++w) acc += red[w];
    }
    if (t == 0) {
      float v = alpha * acc;
      if (y_in != nullptr) v += beta * load_elem(y_in, r, fmt);
      store_elem(y, r, fmt, v);
    }
  }
}

// part[chunk, c] = sum_{r in chunk} A[r, c] * x[r]: the transposed product streams A row by row,
// each thread owning one 16-byte column group; row chunks are folded by splitk_reduce_kernel.
__global__ void gemv_cols_kernel(const void* __restrict__ A, int64_t lda, int fmt, int rows, int cols,
                                 const void* __restrict__ x, float* __restrict__ part, int rows_per_chunk) {
  const int elt = (fmt == FMT_F32) ? 4 : 2;
  const int per = 16 / elt;
  const int cg = blockIdx.x * blockDim.x + threadIdx.x;   // column group
  const int c0 = cg * per;
  if (c0 >= cols) return;
  const int r0 = blockIdx.y * rows_per_chunk;
  const int r1 = min(rows, r0 + rows_per_chunk);
  const bool vec = (c0 + per <= cols) && ((lda * elt) % 16 == 0) && ((reinterpret_cast<uintptr_t>(A) & 15) == 0);
  float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  int r = r0;
  if (vec) {
    // eight rows per step: their loads are independent, so eight 16-byte requests are in flight per thread
    const uint8_t* col = static_cast<const uint8_t*>(A) + static_cast<int64_t>(c0) * elt;
    const int64_t pitch = lda * elt;
    for (; r + 8 <= r1; r += 8) {
      uint4 w[8];
      float xv[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        w[j] = ldg_v4(col + (r + j) * pitch);
        xv[j] = load_elem(x, r + j, fmt);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float fa[8];
        unpack_word(w[j], fmt, fa);
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (i < per) acc[i] += fa[i] * xv[j];
      }
    }
  }
  for (; r < r1; ++r) {
    const float xv = load_elem(x, r, fmt);
    const uint8_t* row = static_cast<const uint8_t*>(A) + static_cast<int64_t>(r) * lda * elt;
    if (vec) {
      float fa[8];
      unpack_word(ldg_v4(row + static_cast<int64_t>(c0) * elt), fmt, fa);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (i < per) acc[i] += fa[i] * xv;
    } else {
      for (int i = 0; i < per && c0 + i < cols; ++i) acc[i] += load_elem(row, c0 + i, fmt) * xv;
    }
  }
  float* dst = part + static_cast<int64_t>(blockIdx.y) * cols + c0;
  for (int i = 0; i < per && c0 + i < cols; ++i) dst[i] = acc[i];
}

bool float_fmt(int fmt) { return fmt == CATCOC_FMT_F16 || fmt == CATCOC_FMT_BF16 || fmt == CATCOC_FMT_F32; }

}  // namespace

extern "C" int catcoc_splitk_reduce(const float* parts, int slices, int64_t slice_elems, int rows, int cols, void* out,
                                    int64_t ldc, int out_fmt, float alpha, float beta, const void* c_src,
                                    int64_t ldc_src, const float* bias, void* stream) {
  if (parts == nullptr || out == nullptr || slices <= 0 || rows <= 0 || cols <= 0 || !float_fmt(out_fmt) ||
      ldc < cols || (c_src != nullptr && ldc_src < cols)) {
    host::set_error("splitk_reduce: bad argument");
    return CATCOC_E_BAD_ARG;
  }
  if ((reinterpret_cast<uintptr_t>(parts) & 15) != 0 || (slice_elems % 4) != 0) {
    host::set_error("splitk_reduce: partial slices must be 16-byte aligned");
    return CATCOC_E_ALIGNMENT;
  }
  const int64_t units = static_cast<int64_t>(rows) * ((cols % 4) == 0 ? cols / 4 : cols);
  int64_t blocks = (units + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      parts, slices, slice_elems, rows, cols, out, ldc, out_fmt, alpha, beta != 0.f ? beta : 0.f,
      beta != 0.f ? c_src : nullptr, ldc_src, bias);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}

extern "C" int64_t catcoc_gemv_workspace_floats(int rows, int cols, int trans) {
  if (!trans) return 0;
  const int chunks = (rows + 127) / 128;
  return static_cast<int64_t>(chunks) * cols;
}

extern "C" int catcoc_gemv(const void* A, int64_t lda, int fmt, int rows, int cols, int trans, const void* x, void* y,
                           const void* y_in, float alpha, float beta, float* workspace, void* stream) {
  if (A == nullptr || x == nullptr || y == nullptr || rows <= 0 || cols <= 0 || lda < cols || !float_fmt(fmt)) {
    host::set_error("gemv: bad argument");
    return CATCOC_E_BAD_ARG;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (beta == 0.f) y_in = nullptr;
  if (!trans) {
    // enough rows to fill the GPU with one warp each, otherwise a block per row
    if (rows >= 148 * 8) {
      const int blocks = (rows + 7) / 8 < 148 * 8 ? (rows + 7) / 8 : 148 * 8;
      gemv_rows_kernel<32><<<blocks, 256, 0, st>>>(A, lda, fmt, rows, cols, x, y, y_in, alpha, beta);
    } else {
      gemv_rows_kernel<256><<<rows, 256, 0, st>>>(A, lda, fmt, rows, cols, x, y, y_in, alpha, beta);
    }
    CATCOC_CUDA_OK(cudaGetLastError());
    return CATCOC_OK;
  }
  if (workspace == nullptr) { host::set_error("gemv: the transposed product needs its workspace"); return CATCOC_E_BAD_ARG; }
  const int elt = (fmt == CATCOC_FMT_F32) ? 4 : 2;
  const int per = 16 / elt;
  const int col_groups = (cols + per - 1) / per;
  // Row chunks of at least 128 rows (what the workspace is sized for), longer when that still leaves about six blocks
  // per SM: fewer partial rows to write and fold.
  const int col_blocks = (col_groups + 127) / 128;
  int want_chunks = (148 * 6 + col_blocks - 1) / col_blocks;
  if (want_chunks < 1) want_chunks = 1;
  int rpc = ((rows + want_chunks - 1) / want_chunks + 7) / 8 * 8;
  if (rpc < 128) rpc = 128;
  const int chunks = (rows + rpc - 1) / rpc;
  dim3 grid(col_blocks, chunks, 1);
  gemv_cols_kernel<<<grid, 128, 0, st>>>(A, lda, fmt, rows, cols, x, workspace, rpc);
  CATCOC_CUDA_OK(cudaGetLastError());
  // y = alpha * sum_chunks part + beta * y_in, as a [1, cols] split-K reduction
  const int64_t slice = cols;   // a width that is not a multiple of 4 is reduced with scalar loads
  const int64_t units = (cols % 4) == 0 ? cols / 4 : cols;
  int64_t blocks = (units + 255) / 256;
  splitk_reduce_kernel<<<static_cast<int>(blocks), 256, 0, st>>>(workspace, chunks, slice, 1, cols, y, cols, fmt, alpha,
                                                                  beta, y_in, cols, nullptr);
  CATCOC_CUDA_OK(cudaGetLastError());
  return CATCOC_OK;
}
