// K2a: row gather OUT[i,:] = X[idx[i],:] (send-buffer fill of the halo exchange), sm_100a.
// G = smallest power of two >= min(32, F/4) lanes copy one row with 128-bit loads, so a
// warp moves 32/G rows per instruction; HBM traffic per row: 4 (index) + 4F read + 4F written.
#include "common.cuh"

namespace gnnagg {

template <bool VEC>
__global__ void __launch_bounds__(256)
    gather_rows_kernel(const float *__restrict__ X, int64_t ldx, const int32_t *__restrict__ idx, int64_t rows, int FV,
                       int log2g, float *__restrict__ OUT, int64_t ldo) {
    const int G = 1 << log2g;
    const int gl = threadIdx.x & (G - 1);
    const int64_t groups_per_block = blockDim.x >> log2g;
    const int64_t stride = groups_per_block * gridDim.x;
    for (int64_t i = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> log2g); i < rows; i += stride) {
        const int64_t src = idx[i];
        if (VEC) {
            const float4 *xp = reinterpret_cast<const float4 *>(X + src * ldx);
            float4 *op = reinterpret_cast<float4 *>(OUT + i * ldo);
            for (int vi = gl; vi < FV; vi += G) op[vi] = __ldg(xp + vi);
        } else {
            const float *xp = X + src * ldx;
            float *op = OUT + i * ldo;
            for (int vi = gl; vi < FV; vi += G) op[vi] = __ldg(xp + vi);
        }
    }
}

}  // namespace gnnagg

using namespace gnnagg;

extern "C" int gnnagg_gather_rows_f32(const float *X, int64_t ldx, const int32_t *idx, int64_t rows, int32_t F,
                                      float *OUT, int64_t ldo, void *stream) {
    if (rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "gather_rows: negative size");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (X == nullptr || idx == nullptr || OUT == nullptr || ldx < F || ldo < F)
        return fail(GNNAGG_ERR_ARG, "gather_rows: null pointer or leading dimension smaller than F");
    const bool vec = (F % 4 == 0) && (ldx % 4 == 0) && (ldo % 4 == 0) && aligned16(X) && aligned16(OUT);
    const int fv = vec ? F / 4 : F;
    int log2g = 0;
    while ((1 << log2g) < fv && log2g < 5) ++log2g;
    const int64_t groups_per_block = 256 >> log2g;
    int64_t blocks = div_up(rows, groups_per_block);
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (vec)
        gather_rows_kernel<true><<<(unsigned)blocks, 256, 0, st>>>(X, ldx, idx, rows, fv, log2g, OUT, ldo);
    else
        gather_rows_kernel<false><<<(unsigned)blocks, 256, 0, st>>>(X, ldx, idx, rows, fv, log2g, OUT, ldo);
    return check_launch("gather_rows_kernel");
}

namespace gnnagg {

// Y[i,:] = X[i,:] * s[i] (+ bias)  (DIV: X[i,:] / s[i], the IEEE quotient): the per-row degree scalings
// around the aggregation (out /= in_degrees; d^-1/2 on either side of the GCN aggregation, where the
// layer's bias rides along).  One lane group per row, 128-bit accesses; Y may alias X.
template <bool VEC, bool DIV>
__global__ void __launch_bounds__(256)
    scale_rows_kernel(const float *X, int64_t ldx, const float *__restrict__ s, const float *__restrict__ bias,
                      int64_t rows, int FV, int log2g, float *Y, int64_t ldy) {
    const int G = 1 << log2g;
    const int gl = threadIdx.x & (G - 1);
    const int64_t groups_per_block = blockDim.x >> log2g;
    const int64_t stride = groups_per_block * gridDim.x;
    for (int64_t i = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> log2g); i < rows; i += stride) {
        const float f = __ldg(s + i);
        if (VEC) {
            const float4 *xp = reinterpret_cast<const float4 *>(X + i * ldx);
            float4 *yp = reinterpret_cast<float4 *>(Y + i * ldy);
            for (int vi = gl; vi < FV; vi += G) {
                float4 v = xp[vi];
                if (DIV) {
                    v.x = __fdiv_rn(v.x, f), v.y = __fdiv_rn(v.y, f), v.z = __fdiv_rn(v.z, f), v.w = __fdiv_rn(v.w, f);
                } else {
                    v.x *= f, v.y *= f, v.z *= f, v.w *= f;
                }
                if (bias != nullptr) {
                    const float4 b = __ldg(reinterpret_cast<const float4 *>(bias) + vi);
                    v.x += b.x, v.y += b.y, v.z += b.z, v.w += b.w;
                }
                yp[vi] = v;
            }
        } else {
            for (int vi = gl; vi < FV; vi += G) {
                const float v = DIV ? __fdiv_rn(X[i * ldx + vi], f) : X[i * ldx + vi] * f;
                Y[i * ldy + vi] = bias != nullptr ? v + __ldg(bias + vi) : v;
            }
        }
    }
}

}  // namespace gnnagg

extern "C" int gnnagg_scale_rows_f32(const float *X, int64_t ldx, const float *s, int64_t rows, int32_t F,
                                     int32_t divide, const float *bias, float *Y, int64_t ldy, void *stream) {
    if (rows < 0 || F < 0 || (divide != 0 && divide != 1)) return fail(GNNAGG_ERR_ARG, "scale_rows: bad size or flag");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (X == nullptr || s == nullptr || Y == nullptr || ldx < F || ldy < F)
        return fail(GNNAGG_ERR_ARG, "scale_rows: null pointer or leading dimension smaller than F");
    const bool vec = (F % 4 == 0) && (ldx % 4 == 0) && (ldy % 4 == 0) && aligned16(X) && aligned16(Y) &&
                     (bias == nullptr || aligned16(bias));
    const int fv = vec ? F / 4 : F;
    int log2g = 0;
    while ((1 << log2g) < fv && log2g < 5) ++log2g;
    const int64_t groups_per_block = 256 >> log2g;
    int64_t blocks = div_up(rows, groups_per_block);
    const int64_t cap = (int64_t)kNumSMs * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
#define LAUNCH(V, D) scale_rows_kernel<V, D><<<(unsigned)blocks, 256, 0, st>>>(X, ldx, s, bias, rows, fv, log2g, Y, ldy)
    if (vec) {
        if (divide) LAUNCH(true, true); else LAUNCH(true, false);
    } else {
        if (divide) LAUNCH(false, true); else LAUNCH(false, false);
    }
#undef LAUNCH
    return check_launch("scale_rows_kernel");
}
