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
