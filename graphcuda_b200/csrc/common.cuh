// Shared helpers for the C-ABI translation units.
#pragma once

#include <cuda_runtime.h>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "../../include/graphcuda_b200.h"

namespace gc {

// Records a thread-local message and returns `code` so call sites can
// `return gc::fail(GC_ERR_INVALID, "...")`.
int fail(int code, const char* fmt, ...);

inline cudaStream_t as_stream(void* s) { return reinterpret_cast<cudaStream_t>(s); }

// Process-wide count of kernel launches issued by this library (gc_launch_count()).
void count_launches(int n);

inline int check_launch(const char* what, int launches = 1) {
  count_launches(launches);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(GC_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return GC_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs

inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

}  // namespace gc

#define GC_REQUIRE(cond, ...)                                   \
  do {                                                          \
    if (!(cond)) return gc::fail(GC_ERR_INVALID, __VA_ARGS__);  \
  } while (0)
