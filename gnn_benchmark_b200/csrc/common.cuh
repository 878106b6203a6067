// Shared host/device helpers of libgnnagg (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "gnnagg.h"

#if defined(__CUDA_ARCH__) && (__CUDA_ARCH__ < 1000)
#error "libgnnagg is written for sm_100a (B200) only"
#endif

namespace gnnagg {

constexpr int kNumSMs = 148;  // B200: 2 dies x 74 SMs; grids are sized in multiples of this
constexpr unsigned kFullMask = 0xffffffffu;

// Records a message for gnnagg_error_string and returns `code`.
int fail(int code, const char *fmt, ...);

// cudaGetLastError() -> status code.
int check_launch(const char *what);

__host__ __device__ inline int64_t div_up(int64_t a, int64_t b) { return (a + b - 1) / b; }

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Gathered feature rows: read-only path, default L2 policy so that hub rows stay resident.
__device__ __forceinline__ float4 ld_nc_v4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float ld_nc(const float *p) { return __ldg(p); }

// Index / value streams and outputs are touched once: evict-first so they do not push
// gathered feature rows out of L2.
__device__ __forceinline__ int32_t ld_stream(const int32_t *p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream_v4(float *p, float4 v) { __stcs(reinterpret_cast<float4 *>(p), v); }
__device__ __forceinline__ void st_stream(float *p, float v) { __stcs(p, v); }

}  // namespace gnnagg
