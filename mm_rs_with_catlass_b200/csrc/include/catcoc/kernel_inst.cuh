// Instantiation units of the fused kernel. Every (operand kind, CTA flavour) pair is compiled in
// a translation unit of its own (kernels/inst/*.cu), so that the build can run them in parallel,
// and comes in up to three epilogue variants chosen at launch:
//   EPI_PLAIN   convert and store only (local GEMM, all-gather GEMM)
//   EPI_REDUCE  + the owner-side fold of the peers' partial tiles (reduce-scatter, all-reduce)
//   EPI_FULL    + int32 bias, per-row / per-column scales, alpha / beta / C / fp32 bias
//   EPI_PULL    16-bit kinds only: partial tiles stay local, reducer warps sum them through the switch
// The variants exist because the optional stages, although skipped at run time, slow the plain
// path down measurably (code size and register pressure in the epilogue warps).
#pragma once
#include <cstring>

#include "catcoc/fused_gemm.cuh"

namespace catcoc {
namespace inst {

// What a translation unit exports for its (kind, flavour).
struct Unit {
  cudaError_t (*prepare)();                                                        // smem attributes
  cudaError_t (*launch)(int epi, const FusedParams& p, int grid, int threads, cudaStream_t s);   // epi: EPI_*
  int (*max_clusters)();                                                           // pair flavour: resident 2-CTA clusters
};

template <int KIND, bool CTA2, int EPI>
cudaError_t set_smem_attr() {
  return cudaFuncSetAttribute(fused_gemm_kernel<KIND, CTA2, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                              Geo<CTA2>::kSmemBytes);
}

template <int KIND, bool CTA2, int EPI>
cudaError_t launch_one(const FusedParams& p, int grid, int threads, cudaStream_t stream) {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(grid, 1, 1);
  // the variants with communication warps may be launched with fewer of them (threads = 0: all)
  const int max_threads = threads_for(EPI);
  cfg.blockDim = dim3((threads >= kThreads && threads <= max_threads && threads % 32 == 0) ? threads : max_threads, 1, 1);
  cfg.dynamicSmemBytes = Geo<CTA2>::kSmemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  if (CTA2) {
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
  }
  return cudaLaunchKernelEx(&cfg, fused_gemm_kernel<KIND, CTA2, EPI>, p);
}

template <int KIND, int EPI>
int query_clusters() {
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = dim3(2, 1, 1);
  cfg.blockDim = dim3(threads_for(EPI), 1, 1);
  cfg.dynamicSmemBytes = Geo<true>::kSmemBytes;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  int n = 0;
  if (cudaOccupancyMaxActiveClusters(&n, fused_gemm_kernel<KIND, true, EPI>, &cfg) != cudaSuccess || n <= 0) {
    cudaGetLastError();
    n = 0;
  }
  return n;
}

// The units (defined in kernels/inst/*.cu).
const Unit& unit_f16_single();
const Unit& unit_f16_pair();
const Unit& unit_i8_single();
const Unit& unit_i8_pair();
const Unit& unit_f8_single();
const Unit& unit_f8_pair();
const Unit& unit_mx_single();

}  // namespace inst
}  // namespace catcoc

// Defines unit_<NAME>() with all three epilogue variants.
#define CATCOC_DEFINE_UNIT_3(NAME, KIND, CTA2)                                                        \
  namespace catcoc { namespace inst {                                                                 \
  static cudaError_t NAME##_prepare() {                                                               \
    cudaError_t e = set_smem_attr<KIND, CTA2, EPI_PLAIN>();                                           \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_REDUCE>();                                \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_FULL>();                                  \
    return e;                                                                                         \
  }                                                                                                   \
  static cudaError_t NAME##_launch(int epi, const FusedParams& p, int grid, int threads, cudaStream_t s) {         \
    if (epi == EPI_PLAIN) return launch_one<KIND, CTA2, EPI_PLAIN>(p, grid, threads, s);                       \
    if (epi == EPI_REDUCE) return launch_one<KIND, CTA2, EPI_REDUCE>(p, grid, threads, s);                     \
    return launch_one<KIND, CTA2, EPI_FULL>(p, grid, threads, s);                                              \
  }                                                                                                   \
  static int NAME##_clusters() { return CTA2 ? query_clusters<KIND, EPI_FULL>() : 0; }                \
  const Unit& unit_##NAME() {                                                                         \
    static const Unit u = {NAME##_prepare, NAME##_launch, NAME##_clusters};                           \
    return u;                                                                                         \
  }                                                                                                   \
  } }

// Four variants: the three above and the pull flavour of reduce-scatter / all-reduce.
#define CATCOC_DEFINE_UNIT_4(NAME, KIND, CTA2)                                                        \
  namespace catcoc { namespace inst {                                                                 \
  static cudaError_t NAME##_prepare() {                                                               \
    cudaError_t e = set_smem_attr<KIND, CTA2, EPI_PLAIN>();                                           \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_REDUCE>();                                \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_FULL>();                                  \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_PULL>();                                  \
    return e;                                                                                         \
  }                                                                                                   \
  static cudaError_t NAME##_launch(int epi, const FusedParams& p, int grid, int threads, cudaStream_t s) { \
    if (epi == EPI_PLAIN) return launch_one<KIND, CTA2, EPI_PLAIN>(p, grid, threads, s);              \
    if (epi == EPI_REDUCE) return launch_one<KIND, CTA2, EPI_REDUCE>(p, grid, threads, s);            \
    if (epi == EPI_PULL) return launch_one<KIND, CTA2, EPI_PULL>(p, grid, threads, s);                \
    return launch_one<KIND, CTA2, EPI_FULL>(p, grid, threads, s);                                     \
  }                                                                                                   \
  static int NAME##_clusters() { return CTA2 ? query_clusters<KIND, EPI_FULL>() : 0; }                \
  const Unit& unit_##NAME() {                                                                         \
    static const Unit u = {NAME##_prepare, NAME##_launch, NAME##_clusters};                           \
    return u;                                                                                         \
  }                                                                                                   \
  } }

// Two variants: plain and full (the full one also serves reduce-only launches).
#define CATCOC_DEFINE_UNIT_2(NAME, KIND, CTA2)                                                        \
  namespace catcoc { namespace inst {                                                                 \
  static cudaError_t NAME##_prepare() {                                                               \
    cudaError_t e = set_smem_attr<KIND, CTA2, EPI_PLAIN>();                                           \
    if (e == cudaSuccess) e = set_smem_attr<KIND, CTA2, EPI_FULL>();                                  \
    return e;                                                                                         \
  }                                                                                                   \
  static cudaError_t NAME##_launch(int epi, const FusedParams& p, int grid, int threads, cudaStream_t s) {         \
    if (epi == EPI_PLAIN) return launch_one<KIND, CTA2, EPI_PLAIN>(p, grid, threads, s);                       \
    return launch_one<KIND, CTA2, EPI_FULL>(p, grid, threads, s);                                              \
  }                                                                                                   \
  static int NAME##_clusters() { return CTA2 ? query_clusters<KIND, EPI_FULL>() : 0; }                \
  const Unit& unit_##NAME() {                                                                         \
    static const Unit u = {NAME##_prepare, NAME##_launch, NAME##_clusters};                           \
    return u;                                                                                         \
  }                                                                                                   \
  } }

// One variant (full) for every launch.
#define CATCOC_DEFINE_UNIT_1(NAME, KIND, CTA2)                                                        \
  namespace catcoc { namespace inst {                                                                 \
  static cudaError_t NAME##_prepare() { return set_smem_attr<KIND, CTA2, EPI_FULL>(); }               \
  static cudaError_t NAME##_launch(int, const FusedParams& p, int grid, int threads, cudaStream_t s) {             \
    return launch_one<KIND, CTA2, EPI_FULL>(p, grid, threads, s);                                              \
  }                                                                                                   \
  static int NAME##_clusters() { return 0; }                                                          \
  const Unit& unit_##NAME() {                                                                         \
    static const Unit u = {NAME##_prepare, NAME##_launch, NAME##_clusters};                           \
    return u;                                                                                         \
  }                                                                                                   \
  } }
