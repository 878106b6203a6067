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

// A set-up step that has to run once per device of the process (function attributes are per
// device): run(f) calls f() the first time it is reached with a given device current and returns
// f's result, cudaSuccess afterwards.  A failed f is retried by the next call.
struct PerDeviceOnce {
    static constexpr int kMaxDevices = 64;
    int done[kMaxDevices] = {0};
    template <typename Fn>
    cudaError_t run(Fn f) {
        int dev = -1;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        if (dev < 0 || dev >= kMaxDevices) return cudaErrorInvalidDevice;
        if (__atomic_load_n(&done[dev], __ATOMIC_ACQUIRE)) return cudaSuccess;
        e = f();  // idempotent: two threads racing here set the same attribute
        if (e == cudaSuccess) __atomic_store_n(&done[dev], 1, __ATOMIC_RELEASE);
        return e;
    }
};

// Gathered feature rows: read-only path, default L2 policy so that hub rows stay resident.
__device__ __forceinline__ float4 ld_nc_v4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float ld_nc(const float *p) { return __ldg(p); }

// Index / value streams and outputs are touched once: evict-first so they do not push
// gathered feature rows out of L2.
__device__ __forceinline__ int32_t ld_stream(const int32_t *p) { return __ldcs(p); }
__device__ __forceinline__ float ld_stream(const float *p) { return __ldcs(p); }
__device__ __forceinline__ void st_stream_v4(float *p, float4 v) { __stcs(reinterpret_cast<float4 *>(p), v); }
__device__ __forceinline__ void st_stream(float *p, float v) { __stcs(p, v); }

// Asynchronous 4-byte global -> shared copies (index / value tiles of the SpMM): no register is tied up
// while the data is in flight; a group is complete for the issuing thread after cp_async_wait and for
// the rest of its warp after a __syncwarp() that follows.
__device__ __forceinline__ void cp_async_4(void *smem, const void *gmem) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

constexpr int kMaxSeg = 1024;  // peer segments per call

// Packed-row prefix of the segments into shared memory: pbase[p] = sum_{q<p} ceil(n_q/epb).
__device__ __forceinline__ void build_packed_prefix(const int32_t *__restrict__ seg, int P, int epb, int *pbase,
                                                    int *sseg = nullptr) {
    if (sseg != nullptr)
        for (int p = threadIdx.x; p <= P; p += blockDim.x) sseg[p] = seg[p];
    if (threadIdx.x < 32) {
        const int lane = threadIdx.x;
        int running = 0;
        for (int p0 = 0; p0 < P; p0 += 32) {
            const int p = p0 + lane;
            int cnt = 0;
            if (p < P) cnt = (seg[p + 1] - seg[p] + epb - 1) / epb;
            int incl = cnt;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(kFullMask, incl, off);
                if (lane >= off) incl += t;
            }
            if (p < P) pbase[p] = running + incl - cnt;
            running += __shfl_sync(kFullMask, incl, 31);
        }
        if (lane == 0) pbase[P] = running;
    }
    __syncthreads();
}

// Packed row R -> segment p with pbase[p] <= R < pbase[p+1] (empty segments skipped).
__device__ __forceinline__ int find_segment(const int *pbase, int P, int R) {
    int lo = 0, hi = P - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (pbase[mid] <= R)
            lo = mid;
        else
            hi = mid - 1;
    }
    // several empty segments may share pbase[lo]; the owner is the last one with pbase <= R,
    // which the search above returns because it moves right on equality.
    return lo;
}


}  // namespace gnnagg
