// Host-side helpers shared by the translation units of libcatcoc_b200: thread-local error
// text and lazily resolved CUDA driver entry points (the library links only the CUDA runtime,
// so it also loads on a machine without a driver, e.g. for CPU-only unit tests).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdio>
#include <string>

namespace catcoc {
namespace host {

void set_error(const char* fmt, ...);
const char* last_error();

// Resolves a driver API symbol through the runtime; returns nullptr (and sets the error text)
// when no driver is present.
void* driver_symbol(const char* name);

template <typename Fn>
inline Fn driver_fn(const char* name) {
  return reinterpret_cast<Fn>(driver_symbol(name));
}

#define CATCOC_CUDA_OK(expr)                                                              \
  do {                                                                                    \
    cudaError_t _e = (expr);                                                              \
    if (_e != cudaSuccess) {                                                              \
      ::catcoc::host::set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                                __FILE__, __LINE__);                                      \
      return -1000 - static_cast<int>(_e);                                                \
    }                                                                                     \
  } while (0)

#define CATCOC_CU_OK(expr)                                                                \
  do {                                                                                    \
    CUresult _r = (expr);                                                                 \
    if (_r != CUDA_SUCCESS) {                                                             \
      ::catcoc::host::set_error("%s failed: CUresult %d (%s:%d)", #expr,                  \
                                static_cast<int>(_r), __FILE__, __LINE__);                \
      return -1000 - static_cast<int>(_r);                                                \
    }                                                                                     \
  } while (0)

}  // namespace host
}  // namespace catcoc
