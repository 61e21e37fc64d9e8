// CPU oracle: naive loops for every product the library computes (plain, affine, matrix-vector,
// batched, grouped along M or K, int8 with int32 accumulation and per-token / per-channel
// dequantisation) and the element-wise acceptance rule. Deliberately simple; it is the ground
// truth the CUDA kernels and the PyTorch goldens are checked against.
//
// Same jobs as the reference's CPU goldens (3rdparty/catlass/examples/common/golden/matmul.hpp:22-368:
// ComputeMatmul, ComputeGemm, ComputeGemv, ComputeGroupGemm, ComputeBatchedMatmul, ComputeGroupedMatmul,
// ComputeMatmulElemWiseAdd, ComputeGroupedMatmulPerTokenDequant, QuantMatmul,
// ComputeGroupedMatmulSliceKPerTokenDequant, ComputeMatmulBias; compare_data.hpp:20-39) and its
// acceptance rule (examples/utils/verify_result.py:106-116). Built differently: every entry point
// below is a thin loop over one strided dot-product helper, and all accumulate wider than the
// device does (double for floats, int64 checked against int32 for integers).
#include <cmath>
#include <cstdint>
#include <limits>
#include "catcoc/capi.h"

namespace {

// A matrix as the oracle sees it: element (r, c) of the LOGICAL matrix lives at base[r * rs + c * cs].
template <typename T>
struct View {
  const T* base;
  int64_t rs, cs;
  T at(int64_t r, int64_t c) const { return base[r * rs + c * cs]; }
};
// logical [rows, cols]; `trans` means the storage holds the transpose row-major ([cols, rows])
template <typename T>
View<T> view_of(const T* p, int rows, int cols, int trans) {
  return trans ? View<T>{p, 1, static_cast<int64_t>(rows)} : View<T>{p, static_cast<int64_t>(cols), 1};
}

template <typename T>
double dot_f(const View<T>& a, int64_t i, const View<T>& b, int64_t j, int k0, int k1) {
  double acc = 0.0;
  for (int k = k0; k < k1; ++k) acc += static_cast<double>(a.at(i, k)) * static_cast<double>(b.at(k, j));
  return acc;
}
// exact integer dot product; reports overflow of the int32 accumulator the device uses
bool dot_i(const View<int8_t>& a, int64_t i, const View<int8_t>& b, int64_t j, int k0, int k1, int64_t init,
           int32_t* out) {
  int64_t acc = init;
  for (int k = k0; k < k1; ++k) acc += static_cast<int64_t>(a.at(i, k)) * static_cast<int64_t>(b.at(k, j));
  *out = static_cast<int32_t>(acc);
  return acc >= std::numeric_limits<int32_t>::min() && acc <= std::numeric_limits<int32_t>::max();
}

// group g of a cumulative list covers [begin, end); malformed lists (decreasing, beyond `limit`)
// are clamped like the device does
void group_range(const int32_t* ends, int g, int limit, int* begin, int* end) {
  auto clamp = [limit](int v) { return v < 0 ? 0 : (v > limit ? limit : v); };
  int b = 0;
  for (int q = 0; q < g; ++q) { const int e = clamp(ends[q]); if (e > b) b = e; }
  int e = clamp(ends[g]);
  if (e < b) e = b;
  *begin = b;
  *end = e;
}

}  // namespace

extern "C" int catcoc_oracle_matmul_f32(const float* a, const float* b, float* c, int M, int N, int K, int trans_a,
                                        int trans_b) {
  if (!a || !b || !c || M < 0 || N < 0 || K < 0) return CATCOC_E_BAD_ARG;
  for (int i = 0; i < M; ++i) {
    for (int j = 0; j < N; ++j) {
      double acc = 0.0;  // wider than the device's fp32 accumulate: the oracle is the better value
      for (int k = 0; k < K; ++k) {
        const float av = trans_a ? a[static_cast<int64_t>(k) * M + i] : a[static_cast<int64_t>(i) * K + k];
        const float bv = trans_b ? b[static_cast<int64_t>(j) * K + k] : b[static_cast<int64_t>(k) * N + j];
        acc += static_cast<double>(av) * static_cast<double>(bv);
      }
      c[static_cast<int64_t>(i) * N + j] = static_cast<float>(acc);
    }
  }
  return CATCOC_OK;
}

extern "C" int catcoc_oracle_quant_matmul(const int8_t* a, const int8_t* b, const int32_t* bias, int32_t* acc, int M,
                                          int N, int K, int trans_a, int trans_b) {
  if (!a || !b || !acc || M < 0 || N < 0 || K < 0) return CATCOC_E_BAD_ARG;
  for (int i = 0; i < M; ++i) {
    for (int j = 0; j < N; ++j) {
      int32_t s = bias ? bias[j] : 0;
      for (int k = 0; k < K; ++k) {
        const int32_t av = trans_a ? a[static_cast<int64_t>(k) * M + i] : a[static_cast<int64_t>(i) * K + k];
        const int32_t bv = trans_b ? b[static_cast<int64_t>(j) * K + k] : b[static_cast<int64_t>(k) * N + j];
        s += av * bv;
      }
      acc[static_cast<int64_t>(i) * N + j] = s;
    }
  }
  return CATCOC_OK;
}

extern "C" int catcoc_oracle_dequant(const int32_t* acc, const float* scale_m, const float* scale_n, float* out, int M,
                                     int N) {
  if (!acc || !out) return CATCOC_E_BAD_ARG;
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j)
      out[static_cast<int64_t>(i) * N + j] = static_cast<float>(acc[static_cast<int64_t>(i) * N + j]) *
                                             (scale_n ? scale_n[j] : 1.0f) * (scale_m ? scale_m[i] : 1.0f);
  return CATCOC_OK;
}

// Returns the number of elements violating |out - golden| <= rtol * max(1, |golden|); NaN/Inf
// on either side count as violations unless both sides agree. Also reports the mean relative
// bias sum|out-golden| / sum|golden|.
extern "C" int64_t catcoc_oracle_compare(const float* out, const float* golden, int64_t n, float rtol,
                                         double* mean_rel_bias) {
  int64_t bad = 0;
  double num = 0.0, den = 0.0;
  for (int64_t i = 0; i < n; ++i) {
    const float o = out[i], g = golden[i];
    if (!std::isfinite(o) || !std::isfinite(g)) {
      if (!((std::isnan(o) && std::isnan(g)) || o == g)) ++bad;
      continue;
    }
    const float tol = rtol * std::fmax(1.0f, std::fabs(g));
    if (std::fabs(o - g) > tol) ++bad;
    num += std::fabs(static_cast<double>(o) - g);
    den += std::fabs(static_cast<double>(g));
  }
  if (mean_rel_bias) *mean_rel_bias = den > 0 ? num / den : 0.0;
  return bad;
}

// ---- the rest of the catalogue ---------------------------------------------------------------

// out = alpha * op(A) op(B) + beta * C + bias[col]; C and bias may be null. Row-major [M, N] C / out.
extern "C" int catcoc_oracle_gemm(const float* a, const float* b, const float* c, const float* bias, float* out,
                                  int M, int N, int K, int trans_a, int trans_b, float alpha, float beta) {
  if (!a || !b || !out || M < 0 || N < 0 || K < 0) return CATCOC_E_BAD_ARG;
  const View<float> va = view_of(a, M, K, trans_a), vb = view_of(b, K, N, trans_b);
  for (int i = 0; i < M; ++i)
    for (int j = 0; j < N; ++j) {
      double v = static_cast<double>(alpha) * dot_f(va, i, vb, j, 0, K);
      if (c) v += static_cast<double>(beta) * c[static_cast<int64_t>(i) * N + j];
      if (bias) v += bias[j];
      out[static_cast<int64_t>(i) * N + j] = static_cast<float>(v);
    }
  return CATCOC_OK;
}

// y = alpha * op(A) x + beta * y_in with A row-major [rows, cols]; op = transpose when `trans`.
extern "C" int catcoc_oracle_gemv(const float* a, const float* x, const float* y_in, float* y, int rows, int cols,
                                  int trans, float alpha, float beta) {
  if (!a || !x || !y || rows < 0 || cols < 0) return CATCOC_E_BAD_ARG;
  const int out_n = trans ? cols : rows, red_n = trans ? rows : cols;
  for (int o = 0; o < out_n; ++o) {
    double acc = 0.0;
    for (int r = 0; r < red_n; ++r)
      acc += static_cast<double>(trans ? a[static_cast<int64_t>(r) * cols + o] : a[static_cast<int64_t>(o) * cols + r]) * x[r];
    y[o] = static_cast<float>(alpha * acc + (y_in ? static_cast<double>(beta) * y_in[o] : 0.0));
  }
  return CATCOC_OK;
}

// out[i] = op(A[i]) op(B[i]) for `batch` densely stacked entries.
extern "C" int catcoc_oracle_batched_matmul(const float* a, const float* b, float* out, int batch, int M, int N, int K,
                                            int trans_a, int trans_b) {
  if (!a || !b || !out || batch < 0) return CATCOC_E_BAD_ARG;
  for (int i = 0; i < batch; ++i) {
    const int rc = catcoc_oracle_gemm(a + static_cast<int64_t>(i) * M * K, b + static_cast<int64_t>(i) * K * N, nullptr,
                                      nullptr, out + static_cast<int64_t>(i) * M * N, M, N, K, trans_a, trans_b, 1.0f, 0.0f);
    if (rc != CATCOC_OK) return rc;
  }
  return CATCOC_OK;
}

// Grouped along M: rows [ends[g-1], ends[g]) of A [M_total, K] meet B[g] ([K, N], or [N, K] with trans_b).
// Rows past the last group's end are left untouched.
extern "C" int catcoc_oracle_grouped_matmul(const float* a, const float* b, const int32_t* ends, int groups, float* out,
                                            int M_total, int N, int K, int trans_b) {
  if (!a || !b || !ends || !out || groups < 0) return CATCOC_E_BAD_ARG;
  const View<float> va = view_of(a, M_total, K, 0);
  for (int g = 0; g < groups; ++g) {
    int r0, r1;
    group_range(ends, g, M_total, &r0, &r1);
    const View<float> vb = view_of(b + static_cast<int64_t>(g) * K * N, K, N, trans_b);
    for (int i = r0; i < r1; ++i)
      for (int j = 0; j < N; ++j) out[static_cast<int64_t>(i) * N + j] = static_cast<float>(dot_f(va, i, vb, j, 0, K));
  }
  return CATCOC_OK;
}

// Grouped along K: out[g] = A[:, ks of g] B[ks of g, :] with A stored [K_total, M] (its transpose, as the
// weight-gradient product has it) and B stored [K_total, N]; out is [groups, M, N].
extern "C" int catcoc_oracle_grouped_matmul_slice_k(const float* a, const float* b, const int32_t* ends, int groups,
                                                    float* out, int M, int N, int K_total) {
  if (!a || !b || !ends || !out || groups < 0) return CATCOC_E_BAD_ARG;
  const View<float> va = view_of(a, M, K_total, 1), vb = view_of(b, K_total, N, 0);
  for (int g = 0; g < groups; ++g) {
    int k0, k1;
    group_range(ends, g, K_total, &k0, &k1);
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j)
        out[(static_cast<int64_t>(g) * M + i) * N + j] = static_cast<float>(dot_f(va, i, vb, j, k0, k1));
  }
  return CATCOC_OK;
}

// int8 grouped along M with dequantisation: out[i, j] = float(sum_k a[i,k] b_g[k,j]) * scale_n[g, j] * scale_m[i].
// Returns CATCOC_E_TOO_LARGE if an exact sum leaves the int32 range the device accumulates in.
extern "C" int catcoc_oracle_grouped_quant_matmul(const int8_t* a, const int8_t* b, const int32_t* ends, int groups,
                                                  const float* scale_m, const float* scale_n, float* out, int M_total,
                                                  int N, int K, int trans_b) {
  if (!a || !b || !ends || !out || groups < 0) return CATCOC_E_BAD_ARG;
  const View<int8_t> va = view_of(a, M_total, K, 0);
  bool fits = true;
  for (int g = 0; g < groups; ++g) {
    int r0, r1;
    group_range(ends, g, M_total, &r0, &r1);
    const View<int8_t> vb = view_of(b + static_cast<int64_t>(g) * K * N, K, N, trans_b);
    for (int i = r0; i < r1; ++i)
      for (int j = 0; j < N; ++j) {
        int32_t acc;
        fits = dot_i(va, i, vb, j, 0, K, 0, &acc) && fits;
        out[static_cast<int64_t>(i) * N + j] = static_cast<float>(acc) *
                                               (scale_n ? scale_n[static_cast<int64_t>(g) * N + j] : 1.0f) *
                                               (scale_m ? scale_m[i] : 1.0f);
      }
  }
  return fits ? CATCOC_OK : CATCOC_E_TOO_LARGE;
}

// int8 grouped along K with dequantisation: out[g, i, j] = float(sum_{k in g} a[k,i] b[k,j]) * scale_n[g, j] * scale_m[g, i]
// with A stored [K_total, M] and B stored [K_total, N].
extern "C" int catcoc_oracle_grouped_quant_matmul_slice_k(const int8_t* a, const int8_t* b, const int32_t* ends,
                                                          int groups, const float* scale_m, const float* scale_n,
                                                          float* out, int M, int N, int K_total) {
  if (!a || !b || !ends || !out || groups < 0) return CATCOC_E_BAD_ARG;
  const View<int8_t> va = view_of(a, M, K_total, 1), vb = view_of(b, K_total, N, 0);
  bool fits = true;
  for (int g = 0; g < groups; ++g) {
    int k0, k1;
    group_range(ends, g, K_total, &k0, &k1);
    for (int i = 0; i < M; ++i)
      for (int j = 0; j < N; ++j) {
        int32_t acc;
        fits = dot_i(va, i, vb, j, k0, k1, 0, &acc) && fits;
        out[(static_cast<int64_t>(g) * M + i) * N + j] =
            static_cast<float>(acc) * (scale_n ? scale_n[static_cast<int64_t>(g) * N + j] : 1.0f) *
            (scale_m ? scale_m[static_cast<int64_t>(g) * M + i] : 1.0f);
      }
  }
  return fits ? CATCOC_OK : CATCOC_E_TOO_LARGE;
}

// Independent problems of unrelated shapes, densely packed one after the other (A_i [M_i, K_i], B_i
// [K_i, N_i], C_i and out_i [M_i, N_i], all row-major): out_i = alpha_i A_i B_i + beta_i C_i.
// `mnk` holds 3 ints per problem.
extern "C" int catcoc_oracle_group_gemm(int count, const int32_t* mnk, const float* alphas, const float* betas,
                                        const float* a, const float* b, const float* c, float* out) {
  if (count < 0 || !mnk || !a || !b || !out) return CATCOC_E_BAD_ARG;
  int64_t oa = 0, ob = 0, oc = 0;
  for (int i = 0; i < count; ++i) {
    const int M = mnk[3 * i], N = mnk[3 * i + 1], K = mnk[3 * i + 2];
    const int rc = catcoc_oracle_gemm(a + oa, b + ob, c ? c + oc : nullptr, nullptr, out + oc, M, N, K, 0, 0,
                                      alphas ? alphas[i] : 1.0f, (betas && c) ? betas[i] : 0.0f);
    if (rc != CATCOC_OK) return rc;
    oa += static_cast<int64_t>(M) * K;
    ob += static_cast<int64_t>(K) * N;
    oc += static_cast<int64_t>(M) * N;
  }
  return CATCOC_OK;
}
