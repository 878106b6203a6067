// Device helpers of the halo codec shared by the codec kernels (codec.cu) and the SpMM whose epilogue
// packs its rows (spmm.cu): ordered-integer min / max, the reference's first-zero / NaN rules, the
// encoder, and the register-resident quantise + pack routine.
#pragma once

#include <cuda_bf16.h>
#include <limits.h>

#include "common.cuh"

namespace gnnagg {

constexpr int kCodecWarps = 4;

// Warp min / max of non-NaN floats with one redux.sync each: floats are mapped to integers of the
// same order (negative values have their magnitude bits flipped) and mapped back.  The lane-local
// inputs are never NaN here (they start from +-inf and fminf / fmaxf skip NaNs); the sign of a zero
// result is settled separately by fix_extreme.
__device__ __forceinline__ int float_to_ordered(float v) {
    const int i = __float_as_int(v);
    return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float ordered_to_float(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }
__device__ __forceinline__ float warp_min(float v) {
    return ordered_to_float(__reduce_min_sync(kFullMask, float_to_ordered(v)));
}
__device__ __forceinline__ float warp_max(float v) {
    return ordered_to_float(__reduce_max_sync(kFullMask, float_to_ordered(v)));
}
__device__ __forceinline__ int warp_min_int(int v) { return __reduce_min_sync(kFullMask, v); }

// The reference scans a row from column 0 and replaces min/max only on a strict compare
// (quantization_arm.cpp:93-104): a NaN never replaces, a NaN in column 0 sticks, and of
// several zeros of either sign the first one met is kept.  fminf/fmaxf already skip
// NaNs; the two corrections below restore the rest.  `first_zero_key` is
// (column << 1 | sign bit) of this lane's first element equal to zero, INT_MAX if none.
__device__ __forceinline__ float fix_extreme(float m, float x0, int first_zero_key) {
    if (x0 != x0) return x0;
    if (m == 0.0f) {
        const int key = warp_min_int(first_zero_key);
        return (key & 1) ? -0.0f : 0.0f;
    }
    return m;
}

// Per-row constants of the encoder.  The code is round-half-even(fl((x - zp) / scale)) with a true
// IEEE division.  Dividing costs an order of magnitude more than the rest of the kernel, so the
// quotient is first estimated as (x - zp) * fl(1/scale) (within 2 ulp of the true quotient when
// scale is a normal number well inside the exponent range); only when that estimate lies within 8
// ulp of a rounding boundary k + 0.5 -- where the two could round to different integers -- is the
// exact division done.  Both paths therefore give the integer the exact division gives.
struct RowCodec {
    float zp, scale, rinv;
    bool fast;  // scale in [2^-100, 2^100]: its reciprocal is a normal number with full precision
};
__device__ __forceinline__ RowCodec make_row_codec(float zp, float scale) {
    RowCodec r;
    r.zp = zp, r.scale = scale;
    const float a = fabsf(scale);
    r.fast = (a >= 7.888609e-31f) && (a <= 1.2676506e30f);
    r.rinv = r.fast ? __frcp_rn(scale) : 0.f;
    return r;
}
__device__ __forceinline__ uint32_t encode(float x, const RowCodec &rc, bool signed_cvt) {
    const float d = __fsub_rn(x, rc.zp);
    float q = __fmul_rn(d, rc.rinv);
    const float k = rintf(q);
    const float to_boundary = 0.5f - fabsf(__fsub_rn(q, k));
    const float eps = fmaxf(fabsf(q), 1.0f) * 9.5367431640625e-07f;  // 2^-20 relative: 8 ulp
    if (!rc.fast || !(to_boundary >= eps)) q = __fdiv_rn(d, rc.scale);  // also catches NaN / inf
    return signed_cvt ? (uint32_t)__float2int_rn(q) : __float2uint_rn(q);
}
__device__ __forceinline__ uint32_t encode(float x, float zp, float scale, bool signed_cvt) {
    const float q = __fdiv_rn(__fsub_rn(x, zp), scale);
    // own parameters: unsigned saturating convert (SVE FCVTZU after FRINTN);
    // caller's parameters: signed convert (x86 cvt_roundps_epi32), negative codes keep
    // their two's-complement bits as in the reference.
    return signed_cvt ? (uint32_t)__float2int_rn(q) : __float2uint_rn(q);
}

__device__ __forceinline__ uint32_t bf16_bits(float v) {
    return (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(v));
}

// Exact (true division) encoding of one packed row held in registers: the rarely taken twin of the
// estimate-based loop in quant_pack_vec_kernel; it runs under a warp-uniform branch of its own.
template <int BITS, int NV, int GQ, int ROWS>
__device__ __forceinline__ void quant_exact_rows(const float4 (&xv)[ROWS][NV], const float (&zp)[ROWS],
                                              const float (&sc)[ROWS], int cnt, int gl, int FV, bool signed_cvt,
                                              int sh0, uint32_t (&words)[NV]) {
    constexpr int EPB = 8 / BITS;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (gl + GQ * k < FV) {
#pragma unroll
            for (int t = 0; t < ROWS; ++t) {
                if (t < cnt) {
                    const int sh = ROWS == EPB ? (EPB - 1 - t) * BITS : sh0;
                    b0 |= encode(xv[t][k].x, zp[t], sc[t], signed_cvt) << sh;
                    b1 |= encode(xv[t][k].y, zp[t], sc[t], signed_cvt) << sh;
                    b2 |= encode(xv[t][k].z, zp[t], sc[t], signed_cvt) << sh;
                    b3 |= encode(xv[t][k].w, zp[t], sc[t], signed_cvt) << sh;
                }
            }
        }
        words[k] = (b0 & 255u) | ((b1 & 255u) << 8) | ((b2 & 255u) << 16) | ((b3 & 255u) << 24);
    }
}

// Quantise + pack input rows held in registers (xv[t][k] = float4 number gl + GQ*k of input row i0 + t),
// by the GQ lanes of one group: per-row min / max, parameters, codes, stores.
//   ROWS == 8 / BITS: the rows are the <= EPB rows of packed row R (the stand-alone pack kernel, which
//     loads them from memory) and the packed bytes are written with plain stores;
//   ROWS == 1: one input row whose codes belong at bit position sh0 of its packed row (the SpMM that
//     encodes each row as soon as it is summed); nothing is stored, the shifted codes are returned in
//     `wout` and the caller merges the rows that share a packed row.
template <int BITS, int NV, int GQ, int ROWS = 8 / BITS>
__device__ __forceinline__ void quant_pack_group(const float4 (&xv)[ROWS][NV], int cnt, int i0, int64_t R, int gl,
                                                 unsigned gmask, int lead, int FV, int F, int params_given,
                                                 float *__restrict__ params, uint32_t *__restrict__ params_bf16,
                                                 uint8_t *__restrict__ codes, int sh0 = 0, uint32_t *wout = nullptr) {
    constexpr int EPB = 8 / BITS;
    constexpr float LEVELS = (float)((1 << BITS) - 1);
    float zp[ROWS], rinv[ROWS], sc[ROWS];
    bool fast[ROWS];
#pragma unroll
    for (int t = 0; t < ROWS; ++t) {
        zp[t] = 0.f, sc[t] = 1.f;
        if (t < cnt) {
            if (!params_given) {
                float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);  // +inf, -inf
#pragma unroll
                for (int k = 0; k < NV; ++k)
                    if (gl + GQ * k < FV) {
                        mn = fminf(fminf(mn, xv[t][k].x), fminf(xv[t][k].y, fminf(xv[t][k].z, xv[t][k].w)));
                        mx = fmaxf(fmaxf(mx, xv[t][k].x), fmaxf(xv[t][k].y, fmaxf(xv[t][k].z, xv[t][k].w)));
                    }
                // lanes past the row's end hold +inf / -inf and drop out of the reduction
                mn = ordered_to_float(__reduce_min_sync(gmask, float_to_ordered(mn)));
                mx = ordered_to_float(__reduce_max_sync(gmask, float_to_ordered(mx)));
                const float x0 = __shfl_sync(gmask, xv[t][0].x, lead);
                if (x0 != x0) {  // a NaN in column 0 is never replaced by the reference's scan
                    mn = mx = x0;
                } else if (mn == 0.0f || mx == 0.0f) {
                    // of several zeros of either sign the reference keeps the first one met:
                    // find the first zero column of the row and take its sign
                    int zkey = INT_MAX;
#pragma unroll
                    for (int k = NV - 1; k >= 0; --k) {
                        const int vi = gl + GQ * k;
                        if (vi < FV) {
                            const float e[4] = {xv[t][k].x, xv[t][k].y, xv[t][k].z, xv[t][k].w};
#pragma unroll
                            for (int i = 3; i >= 0; --i)
                                if (e[i] == 0.0f) zkey = ((vi * 4 + i) << 1) | (int)(__float_as_uint(e[i]) >> 31);
                        }
                    }
                    zkey = __reduce_min_sync(gmask, zkey);
                    const float z = (zkey & 1) ? -0.0f : 0.0f;
                    if (mn == 0.0f) mn = z;
                    if (mx == 0.0f) mx = z;
                }
                float s = __fdiv_rn(__fsub_rn(mx, mn), LEVELS);
                if (s == 0.0f) s = 1.0f;
                zp[t] = mn, sc[t] = s;
                if (gl == 0) {
                    *reinterpret_cast<float2 *>(params + (int64_t)(i0 + t) * 2) = make_float2(mn, s);
                    if (params_bf16) params_bf16[i0 + t] = bf16_bits(mn) | (bf16_bits(s) << 16);
                }
            } else {
                zp[t] = params[(int64_t)(i0 + t) * 2];
                sc[t] = params[(int64_t)(i0 + t) * 2 + 1];
                if (gl == 0 && params_bf16) params_bf16[i0 + t] = bf16_bits(zp[t]) | (bf16_bits(sc[t]) << 16);
            }
        }
        const float a = fabsf(sc[t]);
        fast[t] = (a >= 7.888609e-31f) && (a <= 1.2676506e30f);  // 1/scale is a full-precision normal
        rinv[t] = fast[t] ? __frcp_rn(sc[t]) : 0.f;
    }

    // code = round-half-even(fl((x - zp) / scale)), IEEE division.  The quotient is estimated as
    // (x - zp) * fl(1/scale) -- within 2 ulp of the true quotient -- which rounds to the same integer
    // as the exact quotient unless it lies within 8 ulp of a rounding boundary k + 0.5 (or out of the
    // code range, or is not finite).  The whole packed row is encoded from the estimate first; only if
    // some element of the group was that close to a boundary (about one packed row in a hundred for
    // 2-bit codes) is the row encoded again with true divisions, so the hot loop holds no division.
    constexpr float kBound = LEVELS + 1.0f;
    constexpr float kThr = 0.5f - kBound * 9.5367431640625e-07f;  // 0.5 - 2^-20 * bound
    bool unsure = false;
    auto enc_fast = [&](float x, int t) -> uint32_t {
        const float q = __fmul_rn(__fsub_rn(x, zp[t]), rinv[t]);
        const float k = rintf(q);
        unsure = unsure || !((fabsf(__fsub_rn(q, k)) < kThr) && (fabsf(q) <= kBound));
        return params_given ? (uint32_t)__float2int_rn(k) : __float2uint_rn(k);
    };
    uint32_t words[NV];
#pragma unroll
    for (int t = 0; t < ROWS; ++t) unsure = unsure || (t < cnt && !fast[t]);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (gl + GQ * k < FV) {
#pragma unroll
            for (int t = 0; t < ROWS; ++t) {
                if (t < cnt) {
                    const int sh = ROWS == EPB ? (EPB - 1 - t) * BITS : sh0;
                    b0 |= enc_fast(xv[t][k].x, t) << sh;
                    b1 |= enc_fast(xv[t][k].y, t) << sh;
                    b2 |= enc_fast(xv[t][k].z, t) << sh;
                    b3 |= enc_fast(xv[t][k].w, t) << sh;
                }
            }
        }
        words[k] = (b0 & 255u) | ((b1 & 255u) << 8) | ((b2 & 255u) << 16) | ((b3 & 255u) << 24);
    }
    if (__any_sync(gmask, unsure)) {
        quant_exact_rows<BITS, NV, GQ, ROWS>(xv, zp, sc, cnt, gl, FV, params_given != 0, sh0, words);
    }
    if (ROWS == EPB && wout == nullptr) {
        uint32_t *out = reinterpret_cast<uint32_t *>(codes + R * (int64_t)F);
#pragma unroll
        for (int k = 0; k < NV; ++k)
            if (gl + GQ * k < FV) __stcs(out + gl + GQ * k, words[k]);
    } else {
#pragma unroll
        for (int k = 0; k < NV; ++k) wout[k] = (gl + GQ * k < FV) ? words[k] : 0u;
    }

}

}  // namespace gnnagg
