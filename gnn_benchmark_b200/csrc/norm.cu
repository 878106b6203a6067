// dropout -> LayerNorm -> ReLU of the hidden layers as one forward and one backward kernel.
//
// The reference's model runs the three as separate passes over the (rows x F) activations
// (model/DistSAGE.py:49-54); on a GPU each pass is a full trip through HBM.  Here one warp owns a
// row in registers: forward reads X once and writes Y, 4 keep-bits per float4 chunk and the row's
// (mean, rstd); backward reads the upstream gradient and X once, rebuilds the normalised row and the
// ReLU decision with the forward's arithmetic (so Y is not read), writes dX and accumulates the
// column sums for dgamma / dbeta per CTA; a second small kernel adds the per-CTA partials in a fixed
// order (deterministic, no atomics).
//
// Dropout mask: counter-based (Philox-4x32-10 keyed by a caller-supplied 64-bit seed, counter =
// (row, chunk)); element kept with probability 1 - p, kept values scaled by 1 / (1 - p).
#include "common.cuh"

namespace gnnagg {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;

struct Philox {
    uint32_t k0, k1;
    __device__ __forceinline__ uint4 operator()(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3) const {
        uint32_t a = k0, b = k1;
#pragma unroll
        for (int r = 0; r < 10; ++r) {
            const uint32_t hi0 = __umulhi(0xD2511F53u, c0), lo0 = 0xD2511F53u * c0;
            const uint32_t hi1 = __umulhi(0xCD9E8D57u, c2), lo1 = 0xCD9E8D57u * c2;
            c0 = hi1 ^ c1 ^ a;
            c1 = lo1;
            c2 = hi0 ^ c3 ^ b;
            c3 = lo0;
            a += 0x9E3779B9u;
            b += 0xBB67AE85u;
        }
        return make_uint4(c0, c1, c2, c3);
    }
};

// keep-bits of the float4 chunk `chunk` of row `row`: bit i set = element i kept.
__device__ __forceinline__ uint32_t keep_bits(const Philox &rng, int64_t row, int chunk, uint32_t thresh16) {
    const uint4 r = rng((uint32_t)row, (uint32_t)((uint64_t)row >> 32), (uint32_t)chunk, 0x6e6f726du);
    uint32_t bits = 0;
    bits |= ((r.x & 0xFFFFu) >= thresh16) ? 1u : 0u;
    bits |= ((r.x >> 16) >= thresh16) ? 2u : 0u;
    bits |= ((r.y & 0xFFFFu) >= thresh16) ? 4u : 0u;
    bits |= ((r.y >> 16) >= thresh16) ? 8u : 0u;
    return bits;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFullMask, v, off);
    return v;
}

// NV = float4 chunks per lane (F <= 128 * NV).
template <int NV>
__global__ void __launch_bounds__(kNormThreads)
dropout_ln_relu_fwd_kernel(const float *__restrict__ X, int64_t ldx, int64_t rows, int F, const float *__restrict__ gamma,
                           const float *__restrict__ beta, float eps, float keep_scale, uint32_t thresh16, uint32_t k0,
                           uint32_t k1, float *__restrict__ Y, int64_t ldy, uint8_t *__restrict__ mask,
                           float *__restrict__ stats) {
    const int lane = threadIdx.x & 31;
    const int64_t warp0 = (int64_t)blockIdx.x * kNormWarps + (threadIdx.x >> 5);
    const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
    const int chunks = F >> 2;
    const Philox rng{k0, k1};
    float4 g[NV], b[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int c = lane + 32 * j;
        g[j] = c < chunks ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(0, 0, 0, 0);
        b[j] = c < chunks ? __ldg(reinterpret_cast<const float4 *>(beta) + c) : make_float4(0, 0, 0, 0);
    }
    const float inv_f = 1.0f / (float)F;
    for (int64_t row = warp0; row < rows; row += nwarps) {
        float4 v[NV];
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = lane + 32 * j;
            v[j] = make_float4(0, 0, 0, 0);
            if (c < chunks) {
                v[j] = __ldcs(reinterpret_cast<const float4 *>(X + row * ldx) + c);
                if (thresh16 != 0) {
                    const uint32_t kb = keep_bits(rng, row, c, thresh16);
                    v[j].x = (kb & 1u) ? v[j].x * keep_scale : 0.0f;
                    v[j].y = (kb & 2u) ? v[j].y * keep_scale : 0.0f;
                    v[j].z = (kb & 4u) ? v[j].z * keep_scale : 0.0f;
                    v[j].w = (kb & 8u) ? v[j].w * keep_scale : 0.0f;
                    if (mask != nullptr) mask[row * chunks + c] = (uint8_t)kb;
                }
                s += (v[j].x + v[j].y) + (v[j].z + v[j].w);
            }
        }
        const float mean = warp_sum(s) * inv_f;
        float q = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            if (lane + 32 * j < chunks) {
                const float dx = v[j].x - mean, dy = v[j].y - mean, dz = v[j].z - mean, dw = v[j].w - mean;
                q += (dx * dx + dy * dy) + (dz * dz + dw * dw);
            }
        }
        const float rstd = rsqrtf(warp_sum(q) * inv_f + eps);
        if (lane == 0 && stats != nullptr) {
            stats[2 * row] = mean;
            stats[2 * row + 1] = rstd;
        }
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = lane + 32 * j;
            if (c < chunks) {
                float4 y;
                y.x = fmaxf(fmaf((v[j].x - mean) * rstd, g[j].x, b[j].x), 0.0f);
                y.y = fmaxf(fmaf((v[j].y - mean) * rstd, g[j].y, b[j].y), 0.0f);
                y.z = fmaxf(fmaf((v[j].z - mean) * rstd, g[j].z, b[j].z), 0.0f);
                y.w = fmaxf(fmaf((v[j].w - mean) * rstd, g[j].w, b[j].w), 0.0f);
                *(reinterpret_cast<float4 *>(Y + row * ldy) + c) = y;
            }
        }
    }
}

template <int NV>
__global__ void __launch_bounds__(kNormThreads)
dropout_ln_relu_bwd_kernel(const float *__restrict__ GY, int64_t ldg, const float *__restrict__ X, int64_t ldx,
                           const uint8_t *__restrict__ mask, const float *__restrict__ stats,
                           const float *__restrict__ gamma, const float *__restrict__ beta, int64_t rows, int F,
                           float keep_scale, float *__restrict__ GX, int64_t ldgx, float *__restrict__ partial) {
    __shared__ float red[kNormWarps][32 * 4 + 4];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t warp0 = (int64_t)blockIdx.x * kNormWarps + warp;
    const int64_t nwarps = (int64_t)gridDim.x * kNormWarps;
    const int chunks = F >> 2;
    float4 g[NV], b[NV], dg[NV], db[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        const int c = lane + 32 * j;
        g[j] = c < chunks ? __ldg(reinterpret_cast<const float4 *>(gamma) + c) : make_float4(0, 0, 0, 0);
        b[j] = c < chunks ? __ldg(reinterpret_cast<const float4 *>(beta) + c) : make_float4(0, 0, 0, 0);
        dg[j] = make_float4(0, 0, 0, 0);
        db[j] = make_float4(0, 0, 0, 0);
    }
    const float inv_f = 1.0f / (float)F;
    for (int64_t row = warp0; row < rows; row += nwarps) {
        const float mean = __ldg(stats + 2 * row), rstd = __ldg(stats + 2 * row + 1);
        float4 xh[NV], a[NV];
        uint32_t kbits[NV];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = lane + 32 * j;
            xh[j] = make_float4(0, 0, 0, 0);
            a[j] = make_float4(0, 0, 0, 0);
            kbits[j] = 15u;
            if (c < chunks) {
                float4 v = __ldcs(reinterpret_cast<const float4 *>(X + row * ldx) + c);
                const float4 go = __ldcs(reinterpret_cast<const float4 *>(GY + row * ldg) + c);
                if (mask != nullptr) {
                    const uint32_t kb = mask[row * chunks + c];
                    kbits[j] = kb;
                    v.x = (kb & 1u) ? v.x * keep_scale : 0.0f;
                    v.y = (kb & 2u) ? v.y * keep_scale : 0.0f;
                    v.z = (kb & 4u) ? v.z * keep_scale : 0.0f;
                    v.w = (kb & 8u) ? v.w * keep_scale : 0.0f;
                }
                xh[j].x = (v.x - mean) * rstd;
                xh[j].y = (v.y - mean) * rstd;
                xh[j].z = (v.z - mean) * rstd;
                xh[j].w = (v.w - mean) * rstd;
                // ReLU passes the gradient where the forward output was positive (same arithmetic as forward)
                const float gx_ = fmaf(xh[j].x, g[j].x, b[j].x) > 0.0f ? go.x : 0.0f;
                const float gy_ = fmaf(xh[j].y, g[j].y, b[j].y) > 0.0f ? go.y : 0.0f;
                const float gz_ = fmaf(xh[j].z, g[j].z, b[j].z) > 0.0f ? go.z : 0.0f;
                const float gw_ = fmaf(xh[j].w, g[j].w, b[j].w) > 0.0f ? go.w : 0.0f;
                dg[j].x = fmaf(gx_, xh[j].x, dg[j].x);
                dg[j].y = fmaf(gy_, xh[j].y, dg[j].y);
                dg[j].z = fmaf(gz_, xh[j].z, dg[j].z);
                dg[j].w = fmaf(gw_, xh[j].w, dg[j].w);
                db[j].x += gx_;
                db[j].y += gy_;
                db[j].z += gz_;
                db[j].w += gw_;
                a[j] = make_float4(gx_ * g[j].x, gy_ * g[j].y, gz_ * g[j].z, gw_ * g[j].w);
                s1 += (a[j].x + a[j].y) + (a[j].z + a[j].w);
                s2 += (a[j].x * xh[j].x + a[j].y * xh[j].y) + (a[j].z * xh[j].z + a[j].w * xh[j].w);
            }
        }
        s1 = warp_sum(s1) * inv_f;
        s2 = warp_sum(s2) * inv_f;
#pragma unroll
        for (int j = 0; j < NV; ++j) {
            const int c = lane + 32 * j;
            if (c < chunks) {
                float4 o;
                o.x = rstd * (a[j].x - s1 - xh[j].x * s2);
                o.y = rstd * (a[j].y - s1 - xh[j].y * s2);
                o.z = rstd * (a[j].z - s1 - xh[j].z * s2);
                o.w = rstd * (a[j].w - s1 - xh[j].w * s2);
                if (mask != nullptr) {
                    o.x = (kbits[j] & 1u) ? o.x * keep_scale : 0.0f;
                    o.y = (kbits[j] & 2u) ? o.y * keep_scale : 0.0f;
                    o.z = (kbits[j] & 4u) ? o.z * keep_scale : 0.0f;
                    o.w = (kbits[j] & 8u) ? o.w * keep_scale : 0.0f;
                }
                __stcs(reinterpret_cast<float4 *>(GX + row * ldgx) + c, o);
            }
        }
    }
    // per-CTA column sums: warps add up in warp order, one chunk position j at a time
    float *out_g = partial + (int64_t)blockIdx.x * 2 * F;
    float *out_b = out_g + F;
#pragma unroll
    for (int j = 0; j < NV; ++j) {
        for (int pass = 0; pass < 2; ++pass) {
            const float4 v = pass == 0 ? dg[j] : db[j];
            __syncthreads();
            red[warp][lane * 4 + 0] = v.x;
            red[warp][lane * 4 + 1] = v.y;
            red[warp][lane * 4 + 2] = v.z;
            red[warp][lane * 4 + 3] = v.w;
            __syncthreads();
            if (threadIdx.x < 128) {
                float s = 0.0f;
#pragma unroll
                for (int w = 0; w < kNormWarps; ++w) s += red[w][threadIdx.x];
                const int col = (32 * j) * 4 + threadIdx.x;
                if (col < F) (pass == 0 ? out_g : out_b)[col] = s;
            }
        }
    }
}

// dgamma[c] = sum over CTAs of partial[cta][c], dbeta likewise; fixed order.
__global__ void ln_param_grad_kernel(const float *__restrict__ partial, int nblocks, int F, float *__restrict__ dgamma,
                                     float *__restrict__ dbeta) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= 2 * F) return;
    float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
    int i = 0;
    for (; i + 3 < nblocks; i += 4) {
        s0 += partial[(int64_t)(i + 0) * 2 * F + c];
        s1 += partial[(int64_t)(i + 1) * 2 * F + c];
        s2 += partial[(int64_t)(i + 2) * 2 * F + c];
        s3 += partial[(int64_t)(i + 3) * 2 * F + c];
    }
    for (; i < nblocks; ++i) s0 += partial[(int64_t)i * 2 * F + c];
    const float s = (s0 + s1) + (s2 + s3);
    if (c < F)
        dgamma[c] = s;
    else
        dbeta[c - F] = s;
}


// y = relu(x) * keep / (1 - p) in one pass (Y may alias X); mask gets 4 bits per float4 chunk:
// bit i set = element i was positive and kept, i.e. the gradient passes (scaled).  F % 4 == 0.
__global__ void __launch_bounds__(256)
relu_dropout_fwd_kernel(const float *X, int64_t ldx, int64_t rows, int chunks, float keep_scale, uint32_t thresh16,
                        uint32_t k0, uint32_t k1, float *Y, int64_t ldy, uint8_t *__restrict__ mask) {
    const Philox rng{k0, k1};
    const int64_t total = rows * chunks;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / chunks;
        const int c = (int)(i - row * chunks);
        float4 v = *(reinterpret_cast<const float4 *>(X + row * ldx) + c);
        uint32_t kb = thresh16 != 0 ? keep_bits(rng, row, c, thresh16) : 15u;
        kb &= (v.x > 0.0f ? 1u : 0u) | (v.y > 0.0f ? 2u : 0u) | (v.z > 0.0f ? 4u : 0u) | (v.w > 0.0f ? 8u : 0u);
        v.x = (kb & 1u) ? v.x * keep_scale : 0.0f;
        v.y = (kb & 2u) ? v.y * keep_scale : 0.0f;
        v.z = (kb & 4u) ? v.z * keep_scale : 0.0f;
        v.w = (kb & 8u) ? v.w * keep_scale : 0.0f;
        *(reinterpret_cast<float4 *>(Y + row * ldy) + c) = v;
        if (mask != nullptr) mask[i] = (uint8_t)kb;
    }
}

// gx = gy * mask * keep_scale (GX may alias GY).
__global__ void __launch_bounds__(256)
relu_dropout_bwd_kernel(const float *GY, int64_t ldg, const uint8_t *__restrict__ mask, int64_t rows, int chunks,
                        float keep_scale, float *GX, int64_t ldgx) {
    const int64_t total = rows * chunks;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t row = i / chunks;
        const int c = (int)(i - row * chunks);
        float4 v = *(reinterpret_cast<const float4 *>(GY + row * ldg) + c);
        const uint32_t kb = mask[i];
        v.x = (kb & 1u) ? v.x * keep_scale : 0.0f;
        v.y = (kb & 2u) ? v.y * keep_scale : 0.0f;
        v.z = (kb & 4u) ? v.z * keep_scale : 0.0f;
        v.w = (kb & 8u) ? v.w * keep_scale : 0.0f;
        *(reinterpret_cast<float4 *>(GX + row * ldgx) + c) = v;
    }
}

constexpr int kNormGrid = kNumSMs * 8;

int norm_grid(int64_t rows) {
    const int64_t need = div_up(rows, kNormWarps);
    return (int)(need < kNormGrid ? (need < 1 ? 1 : need) : kNormGrid);
}

int check_shape(const char *what, int64_t rows, int F, int64_t ld0, int64_t ld1, const void *p0, const void *p1,
                const void *g, const void *b) {
    if (rows < 0 || F <= 0) return fail(GNNAGG_ERR_ARG, "%s: negative size", what);
    if ((F & 3) != 0 || F > 1024) return fail(GNNAGG_ERR_UNSUPPORTED, "%s: F = %d must be a multiple of 4, at most 1024", what, F);
    if (ld0 < F || ld1 < F || (ld0 & 3) != 0 || (ld1 & 3) != 0)
        return fail(GNNAGG_ERR_UNSUPPORTED, "%s: row strides must be multiples of 4 and at least F", what);
    if (!aligned16(p0) || !aligned16(p1) || !aligned16(g) || !aligned16(b))
        return fail(GNNAGG_ERR_UNSUPPORTED, "%s: operands must be 16-byte aligned", what);
    return GNNAGG_OK;
}

}  // namespace
}  // namespace gnnagg

using namespace gnnagg;

extern "C" size_t gnnagg_dropout_ln_relu_partial_bytes(int32_t F) {
    return F > 0 ? (size_t)kNormGrid * 2 * (size_t)F * sizeof(float) : 0;
}

extern "C" int gnnagg_dropout_ln_relu_fwd(const float *X, int64_t ldx, int64_t rows, int32_t F, const float *gamma,
                                          const float *beta, float eps, float p_drop, uint64_t seed, float *Y,
                                          int64_t ldy, uint8_t *mask, float *stats, void *stream) {
    if (rows == 0) return GNNAGG_OK;
    if (X == nullptr || Y == nullptr || gamma == nullptr || beta == nullptr)
        return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_fwd: null pointer");
    if (!(p_drop >= 0.0f && p_drop < 1.0f)) return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_fwd: p must be in [0,1)");
    int rc = check_shape("dropout_ln_relu_fwd", rows, F, ldx, ldy, X, Y, gamma, beta);
    if (rc != GNNAGG_OK) return rc;
    uint32_t thresh = (uint32_t)(p_drop * 65536.0f + 0.5f);
    if (p_drop > 0.0f && thresh == 0) thresh = 1;
    if (thresh > 0 && mask == nullptr && stats != nullptr)
        return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_fwd: a training call with dropout needs the mask buffer");
    const float keep_scale = thresh ? 65536.0f / (float)(65536u - thresh) : 1.0f;
    const uint32_t k0 = (uint32_t)seed, k1 = (uint32_t)(seed >> 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = norm_grid(rows);
    const int nv = (F + 127) / 128;
#define LAUNCH(NV) \
    dropout_ln_relu_fwd_kernel<NV><<<grid, kNormThreads, 0, st>>>(X, ldx, rows, F, gamma, beta, eps, keep_scale, thresh, k0, k1, Y, ldy, mask, stats)
    if (nv <= 1) LAUNCH(1);
    else if (nv <= 2) LAUNCH(2);
    else if (nv <= 4) LAUNCH(4);
    else LAUNCH(8);
#undef LAUNCH
    return check_launch("dropout_ln_relu_fwd_kernel");
}

extern "C" int gnnagg_dropout_ln_relu_bwd(const float *GY, int64_t ldg, const float *X, int64_t ldx, const uint8_t *mask,
                                          const float *stats, const float *gamma, const float *beta, int64_t rows,
                                          int32_t F, float p_drop, float *GX, int64_t ldgx, float *partial,
                                          size_t partial_bytes, float *dgamma, float *dbeta, void *stream) {
    if (GY == nullptr || X == nullptr || stats == nullptr || gamma == nullptr || beta == nullptr || GX == nullptr ||
        partial == nullptr || dgamma == nullptr || dbeta == nullptr)
        return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_bwd: null pointer");
    if (!(p_drop >= 0.0f && p_drop < 1.0f)) return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_bwd: p must be in [0,1)");
    int rc = check_shape("dropout_ln_relu_bwd", rows, F, ldx, ldg, X, GY, gamma, beta);
    if (rc != GNNAGG_OK) return rc;
    if (ldgx < F || (ldgx & 3) != 0 || !aligned16(GX))
        return fail(GNNAGG_ERR_UNSUPPORTED, "dropout_ln_relu_bwd: dX must be 16-byte aligned with a row stride multiple of 4");
    if (partial_bytes < gnnagg_dropout_ln_relu_partial_bytes(F))
        return fail(GNNAGG_ERR_SCRATCH, "dropout_ln_relu_bwd: partial-sum scratch too small");
    uint32_t thresh = (uint32_t)(p_drop * 65536.0f + 0.5f);
    if (p_drop > 0.0f && thresh == 0) thresh = 1;
    if (thresh > 0 && mask == nullptr) return fail(GNNAGG_ERR_ARG, "dropout_ln_relu_bwd: dropout needs the forward's mask");
    const float keep_scale = thresh ? 65536.0f / (float)(65536u - thresh) : 1.0f;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int grid = rows > 0 ? norm_grid(rows) : 1;
    const int nv = (F + 127) / 128;
    const uint8_t *m = thresh ? mask : nullptr;
#define LAUNCH(NV) \
    dropout_ln_relu_bwd_kernel<NV><<<grid, kNormThreads, 0, st>>>(GY, ldg, X, ldx, m, stats, gamma, beta, rows, F, keep_scale, GX, ldgx, partial)
    if (nv <= 1) LAUNCH(1);
    else if (nv <= 2) LAUNCH(2);
    else if (nv <= 4) LAUNCH(4);
    else LAUNCH(8);
#undef LAUNCH
    rc = check_launch("dropout_ln_relu_bwd_kernel");
    if (rc != GNNAGG_OK) return rc;
    ln_param_grad_kernel<<<(2 * F + 127) / 128, 128, 0, st>>>(partial, grid, F, dgamma, dbeta);
    return check_launch("ln_param_grad_kernel");
}

static uint32_t drop_threshold(float p_drop) {
    uint32_t thresh = (uint32_t)(p_drop * 65536.0f + 0.5f);
    if (p_drop > 0.0f && thresh == 0) thresh = 1;
    return thresh;
}

extern "C" int gnnagg_relu_dropout_fwd(const float *X, int64_t ldx, int64_t rows, int32_t F, float p_drop, uint64_t seed,
                                       float *Y, int64_t ldy, uint8_t *mask, void *stream) {
    if (rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "relu_dropout_fwd: negative size");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (X == nullptr || Y == nullptr) return fail(GNNAGG_ERR_ARG, "relu_dropout_fwd: null pointer");
    if (!(p_drop >= 0.0f && p_drop < 1.0f)) return fail(GNNAGG_ERR_ARG, "relu_dropout_fwd: p must be in [0,1)");
    if ((F & 3) != 0 || (ldx & 3) != 0 || (ldy & 3) != 0 || ldx < F || ldy < F || !aligned16(X) || !aligned16(Y))
        return fail(GNNAGG_ERR_UNSUPPORTED, "relu_dropout_fwd: F and row strides must be multiples of 4, rows 16-byte aligned");
    const uint32_t thresh = drop_threshold(p_drop);
    const float keep_scale = thresh ? 65536.0f / (float)(65536u - thresh) : 1.0f;
    const int64_t total = rows * (F >> 2);
    const int64_t want = div_up(total, 256);
    const int grid = (int)(want < (int64_t)kNumSMs * 16 ? want : (int64_t)kNumSMs * 16);
    relu_dropout_fwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        X, ldx, rows, F >> 2, keep_scale, thresh, (uint32_t)seed, (uint32_t)(seed >> 32), Y, ldy, mask);
    return check_launch("relu_dropout_fwd_kernel");
}

extern "C" int gnnagg_relu_dropout_bwd(const float *GY, int64_t ldg, const uint8_t *mask, int64_t rows, int32_t F,
                                       float p_drop, float *GX, int64_t ldgx, void *stream) {
    if (rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "relu_dropout_bwd: negative size");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (GY == nullptr || GX == nullptr || mask == nullptr) return fail(GNNAGG_ERR_ARG, "relu_dropout_bwd: null pointer");
    if (!(p_drop >= 0.0f && p_drop < 1.0f)) return fail(GNNAGG_ERR_ARG, "relu_dropout_bwd: p must be in [0,1)");
    if ((F & 3) != 0 || (ldg & 3) != 0 || (ldgx & 3) != 0 || ldg < F || ldgx < F || !aligned16(GY) || !aligned16(GX))
        return fail(GNNAGG_ERR_UNSUPPORTED, "relu_dropout_bwd: F and row strides must be multiples of 4, rows 16-byte aligned");
    const uint32_t thresh = drop_threshold(p_drop);
    const float keep_scale = thresh ? 65536.0f / (float)(65536u - thresh) : 1.0f;
    const int64_t total = rows * (F >> 2);
    const int64_t want = div_up(total, 256);
    const int grid = (int)(want < (int64_t)kNumSMs * 16 ? want : (int64_t)kNumSMs * 16);
    relu_dropout_bwd_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(GY, ldg, mask, rows, F >> 2,
                                                                               keep_scale, GX, ldgx);
    return check_launch("relu_dropout_bwd_kernel");
}
