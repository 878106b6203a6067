// Status codes, error text and small element-wise kernels of libgnnagg.
#include <cuda_bf16.h>
#include <stdarg.h>
#include <string.h>

#include "common.cuh"

namespace gnnagg {

static thread_local char g_msg[256] = {0};
static thread_local int g_msg_code = 0;

int fail(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof(g_msg), fmt, ap);
    va_end(ap);
    g_msg_code = code;
    return code;
}

int check_launch(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return GNNAGG_OK;
    return fail(GNNAGG_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
}

__global__ void cast_f32_bf16_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __float2bfloat16_rn(__ldcs(src + i));
}

__global__ void cast_bf16_f32_kernel(const __nv_bfloat16 *__restrict__ src, float *__restrict__ dst, int64_t n) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __bfloat162float(src[i]);
}

}  // namespace gnnagg

using namespace gnnagg;

extern "C" int gnnagg_version(void) { return 100; }

extern "C" const char *gnnagg_error_string(int code) {
    if (code < 0 && code == g_msg_code && g_msg[0] != 0) return g_msg;
    switch (code) {
        case GNNAGG_OK:
            return "ok";
        case GNNAGG_ERR_ARG:
            return "invalid argument";
        case GNNAGG_ERR_UNSUPPORTED:
            return "unsupported shape";
        case GNNAGG_ERR_CUDA:
            return "CUDA launch error";
        case GNNAGG_ERR_SCRATCH:
            return "plan or scratch buffer too small or malformed";
        default:
            return "unknown status";
    }
}

static unsigned grid_for(int64_t n, int threads) {
    int64_t b = div_up(n, threads);
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (b > cap) b = cap;
    if (b < 1) b = 1;
    return (unsigned)b;
}

extern "C" int gnnagg_cast_f32_to_bf16(const float *src, void *dst_bf16, int64_t n, void *stream) {
    if (n < 0 || (n > 0 && (src == nullptr || dst_bf16 == nullptr)))
        return fail(GNNAGG_ERR_ARG, "cast_f32_to_bf16: null pointer or negative size");
    if (n == 0) return GNNAGG_OK;
    cast_f32_bf16_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        src, static_cast<__nv_bfloat16 *>(dst_bf16), n);
    return check_launch("cast_f32_bf16_kernel");
}

extern "C" int gnnagg_cast_bf16_to_f32(const void *src_bf16, float *dst, int64_t n, void *stream) {
    if (n < 0 || (n > 0 && (src_bf16 == nullptr || dst == nullptr)))
        return fail(GNNAGG_ERR_ARG, "cast_bf16_to_f32: null pointer or negative size");
    if (n == 0) return GNNAGG_OK;
    cast_bf16_f32_kernel<<<grid_for(n, 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const __nv_bfloat16 *>(src_bf16), dst, n);
    return check_launch("cast_bf16_f32_kernel");
}
