// CPU oracle: naive triple-loop GEMMs (fp32 and int8 -> int32 accumulate), the per-token /
// per-channel dequantisation and the element-wise acceptance rule. Deliberately simple; it is
// the ground truth the CUDA kernels and the PyTorch goldens are checked against.
//
// Modelled on the reference's CPU goldens (3rdparty/catlass/examples/common/golden/matmul.hpp:22-302,
// compare_data.hpp:20-39) and its acceptance rule (examples/utils/verify_result.py:106-116).
#include <cmath>
#include <cstdint>
#include "catcoc/capi.h"

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
