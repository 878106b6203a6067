// K3: per-row min/max quantise + pack, unpack + dequantise (halo exchange codec), sm_100a.
//
// Row-packed layout (live int2 path and the generic 2/4/8-bit variant): EPB = 8/bits
// consecutive rows of one peer segment share one byte per column, first row in the high
// bits; a segment's packed rows start at base_p = sum_{q<p} ceil(n_q/EPB)
// (model/ops/src/quantization_arm.cpp:21-78,158-166).  One warp owns one packed row:
// it reads its <= EPB input rows once with 128-bit loads, keeps them in registers, finds
// min/max with shuffles, encodes from registers and writes F bytes + the parameters.
// HBM traffic per input row: 4F read, F*bits/8 + 8 (+4 for the bf16 copy) written.
//
// Arithmetic is written with explicit IEEE intrinsics so that codes are bit-identical to
// the reference: subtract, true divide, round-half-even, (x - zp) / scale with
// scale = (max - min) / (2^bits - 1) and scale == 0 -> 1; decode is one fma.
#include <cuda_bf16.h>

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
template <int BITS, int NV, int GQ>
__device__ __forceinline__ void quant_exact_rows(const float4 (&xv)[8 / BITS][NV], const float (&zp)[8 / BITS],
                                              const float (&sc)[8 / BITS], int cnt, int gl, int FV, bool signed_cvt,
                                              uint32_t (&words)[NV]) {
    constexpr int EPB = 8 / BITS;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (gl + GQ * k < FV) {
#pragma unroll
            for (int t = 0; t < EPB; ++t) {
                if (t < cnt) {
                    const int sh = (EPB - 1 - t) * BITS;
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

// Quantise + pack one packed row whose <= EPB input rows are held in registers (xv[t][k] = float4 number
// gl + GQ*k of input row i0 + t), by the GQ lanes of one group: per-row min / max, parameters, codes,
// stores.  Shared by the stand-alone pack kernel (rows loaded from memory) and by the SpMM whose
// epilogue packs the rows it has just summed.
template <int BITS, int NV, int GQ>
__device__ __forceinline__ void quant_pack_group(const float4 (&xv)[8 / BITS][NV], int cnt, int i0, int64_t R, int gl,
                                                 unsigned gmask, int lead, int FV, int F, int params_given,
                                                 float *__restrict__ params, uint32_t *__restrict__ params_bf16,
                                                 uint8_t *__restrict__ codes) {
    constexpr int EPB = 8 / BITS;
    constexpr float LEVELS = (float)((1 << BITS) - 1);
    float zp[EPB], rinv[EPB], sc[EPB];
    bool fast[EPB];
#pragma unroll
    for (int t = 0; t < EPB; ++t) {
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
    for (int t = 0; t < EPB; ++t) unsure = unsure || (t < cnt && !fast[t]);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        uint32_t b0 = 0, b1 = 0, b2 = 0, b3 = 0;
        if (gl + GQ * k < FV) {
#pragma unroll
            for (int t = 0; t < EPB; ++t) {
                if (t < cnt) {
                    const int sh = (EPB - 1 - t) * BITS;
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
        quant_exact_rows<BITS, NV, GQ>(xv, zp, sc, cnt, gl, FV, params_given != 0, words);
    }
    uint32_t *out = reinterpret_cast<uint32_t *>(codes + R * (int64_t)F);
#pragma unroll
    for (int k = 0; k < NV; ++k)
        if (gl + GQ * k < FV) __stcs(out + gl + GQ * k, words[k]);

}

// ---- fast path: F % 4 == 0, F <= 512, 16-byte aligned rows ------------------------------
// GQ lanes own one packed row (GQ = 8, 16 or 32 by width), so a warp works on 32/GQ packed rows at a
// time and narrow rows do not leave lanes idle; NV float4 per lane and input row (NV > 1 only with
// GQ = 32).  Reductions and broadcasts are scoped to the group's lane mask.
template <int BITS, int NV, int GQ>
__global__ void __launch_bounds__(kCodecWarps * 32, (NV == 1 ? 8 : (NV == 2 ? 5 : 3)))
    quant_pack_vec_kernel(const float *__restrict__ X, int64_t ldx, const int32_t *__restrict__ idx, int F,
                          const int32_t *__restrict__ seg, int P, int params_given, float *__restrict__ params,
                          uint32_t *__restrict__ params_bf16, uint8_t *__restrict__ codes) {
    constexpr int EPB = 8 / BITS;
    constexpr int NG = 32 / GQ;
    __shared__ int pbase[kMaxSeg + 1];
    __shared__ int sseg[kMaxSeg + 1];
    build_packed_prefix(seg, P, EPB, pbase, sseg);
    const int lane = threadIdx.x & 31;
    const int gl = lane % GQ, grp = lane / GQ;
    const unsigned gmask = GQ == 32 ? kFullMask : (((1u << GQ) - 1u) << (grp * GQ));
    const int lead = grp * GQ;  // the group's lane that holds column 0
    const int FV = F >> 2;
    const int64_t total = pbase[P];
    const int64_t stride = (int64_t)gridDim.x * kCodecWarps * NG;
    for (int64_t R = ((int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5)) * NG + grp; R < total; R += stride) {
        const int p = find_segment(pbase, P, (int)R);
        const int i0 = sseg[p] + ((int)R - pbase[p]) * EPB;
        const int cnt = min(EPB, sseg[p + 1] - i0);

        float4 xv[EPB][NV];
        const float *xp[EPB];
#pragma unroll
        for (int t = 0; t < EPB; ++t) {  // all loads of the group first: EPB*NV independent 16-byte loads per lane
            xp[t] = X;
            if (t < cnt) xp[t] = X + (idx ? (int64_t)idx[i0 + t] : (int64_t)(i0 + t)) * ldx;
        }
#pragma unroll
        for (int t = 0; t < EPB; ++t)
#pragma unroll
            for (int k = 0; k < NV; ++k) {
                const int vi = gl + GQ * k;
                xv[t][k] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < cnt && vi < FV) xv[t][k] = __ldcs(reinterpret_cast<const float4 *>(xp[t]) + vi);
            }

        quant_pack_group<BITS, NV, GQ>(xv, cnt, i0, R, gl, gmask, lead, FV, F, params_given, params, params_bf16,
                                       codes);
    }
}

// ---- rows far longer than one lane group should sum alone (hub vertices) -------------------
// The fused SpMM + pack kernel gives a packed row to one lane group, which is right for the short rows
// of a halo matrix and hopeless for a hub with 10^5 nonzeros.  Rows above kLongRow nonzeros are
// therefore summed beforehand: the row is cut into segments of kLongSeg nonzeros, one CTA per segment
// (its four warps take a quarter each and are folded in warp order), and a second kernel adds a row's
// segment sums in segment order.  Deterministic; long rows differ from the sequential chain by fp32
// re-association only (as rows cut across chunks do in the plain SpMM).
constexpr int kLongSeg = 4096;

template <int NV, int U>
__global__ void __launch_bounds__(128)
    spmm_long_rows_partial_kernel(const int64_t *__restrict__ rowptr, const int32_t *__restrict__ col,
                                  const float *__restrict__ val, const float *__restrict__ X, int64_t ldx, int FV,
                                  const int32_t *__restrict__ long_idx, const int32_t *__restrict__ seg_row,
                                  const int32_t *__restrict__ seg_off, float *__restrict__ partial, int64_t ld) {
    __shared__ float4 fold[3][NV * 32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int s = blockIdx.x;
    const int row = long_idx[seg_row[s]];
    const int64_t r0 = rowptr[row] + (int64_t)seg_off[s] * kLongSeg;
    int64_t r1 = r0 + kLongSeg;
    if (r1 > rowptr[row + 1]) r1 = rowptr[row + 1];
    const int64_t e0 = r0 + (int64_t)warp * (kLongSeg / 4);
    int64_t e1 = e0 + kLongSeg / 4;
    if (e1 > r1) e1 = r1;
    float4 acc[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) acc[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int64_t eb = e0; eb < e1; eb += 32) {
        const int nb = (int)((e1 - eb) < 32 ? (e1 - eb) : 32);
        int my_col = 0;
        float my_val = 0.f;
        if (lane < nb) {
            my_col = ld_stream(col + eb + lane);
            my_val = ld_stream(val + eb + lane);
        }
        for (int j0 = 0; j0 < nb; j0 += U) {
            float4 xr[U][NV];
            float av[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = j0 + u;
                const int c = __shfl_sync(kFullMask, my_col, j & 31);
                av[u] = __shfl_sync(kFullMask, my_val, j & 31);
                const float4 *xp = reinterpret_cast<const float4 *>(X + (int64_t)c * ldx);
#pragma unroll
                for (int k = 0; k < NV; ++k)
                    if (j < nb && lane + 32 * k < FV) xr[u][k] = __ldg(xp + lane + 32 * k);
            }
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (j0 + u < nb) {
#pragma unroll
                    for (int k = 0; k < NV; ++k)
                        if (lane + 32 * k < FV) {
                            acc[k].x = fmaf(av[u], xr[u][k].x, acc[k].x);
                            acc[k].y = fmaf(av[u], xr[u][k].y, acc[k].y);
                            acc[k].z = fmaf(av[u], xr[u][k].z, acc[k].z);
                            acc[k].w = fmaf(av[u], xr[u][k].w, acc[k].w);
                        }
                }
        }
    }
    if (warp > 0) {
#pragma unroll
        for (int k = 0; k < NV; ++k) fold[warp - 1][k * 32 + lane] = acc[k];
    }
    __syncthreads();
    if (warp == 0) {
        float4 *out = reinterpret_cast<float4 *>(partial + (int64_t)s * ld);
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            if (lane + 32 * k < FV) {
                float4 a = acc[k];
#pragma unroll
                for (int w = 0; w < 3; ++w) {
                    const float4 b = fold[w][k * 32 + lane];
                    a.x += b.x, a.y += b.y, a.z += b.z, a.w += b.w;
                }
                out[lane + 32 * k] = a;
            }
        }
    }
}

__global__ void __launch_bounds__(128)
    spmm_long_rows_reduce_kernel(const int32_t *__restrict__ row_seg_ptr, int L, const float *__restrict__ partial,
                                 float *__restrict__ sums, int64_t ld, int F) {
    const int k = blockIdx.x;
    if (k >= L) return;
    const int s0 = row_seg_ptr[k], s1 = row_seg_ptr[k + 1];
    for (int f = threadIdx.x; f < F; f += blockDim.x) {
        float a = 0.f;
        for (int s = s0; s < s1; ++s) a += partial[(int64_t)s * ld + f];
        sums[(int64_t)k * ld + f] = a;
    }
}

// ---- K2 + K3a fused: SpMM whose epilogue quantises + packs -------------------------------
// Row i of the sparse matrix is wire slot i (the send side of the pre/post scheme,
// adj_t_pre_post_aggr_to, or the transposed receive-side matrix in backward).  The GQ lanes that
// own a packed row sum its <= EPB slot rows one after the other -- one fused multiply-add per
// nonzero in CSR order, starting from zero: the reference's chain (model/ops/src/spmm.cpp:97-126)
// -- keep the sums in registers and hand them to quant_pack_group, so the fp32 send buffer is never
// written to or read from HBM.  Column indices / values are read GQ at a time (coalesced) and
// broadcast inside the group; EPB * U gathers are in flight per lane.
template <int BITS, int NV, int GQ, int U>
__global__ void __launch_bounds__(kCodecWarps * 32)
    spmm_quant_pack_kernel(const int64_t *__restrict__ rowptr, const int32_t *__restrict__ col,
                           const float *__restrict__ val, const float *__restrict__ X, int64_t ldx, int F,
                           const int32_t *__restrict__ seg, int P, const int32_t *__restrict__ long_pos,
                           const float *__restrict__ long_sums, int64_t ld_long, float *__restrict__ params,
                           uint32_t *__restrict__ params_bf16, uint8_t *__restrict__ codes) {
    constexpr int EPB = 8 / BITS;
    constexpr int NG = 32 / GQ;
    __shared__ int pbase[kMaxSeg + 1];
    __shared__ int sseg[kMaxSeg + 1];
    build_packed_prefix(seg, P, EPB, pbase, sseg);
    const int lane = threadIdx.x & 31;
    const int gl = lane % GQ, grp = lane / GQ;
    const unsigned gmask = GQ == 32 ? kFullMask : (((1u << GQ) - 1u) << (grp * GQ));
    const int lead = grp * GQ;
    const int FV = F >> 2;
    const int64_t R = ((int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5)) * NG + grp;
    if (R >= pbase[P]) return;  // whole groups leave together: every later shuffle names the group's lanes only
    const int p = find_segment(pbase, P, (int)R);
    const int i0 = sseg[p] + ((int)R - pbase[p]) * EPB;
    const int cnt = min(EPB, sseg[p + 1] - i0);

    float4 acc[EPB][NV];
#pragma unroll
    for (int t = 0; t < EPB; ++t)
#pragma unroll
        for (int k = 0; k < NV; ++k) acc[t][k] = make_float4(0.f, 0.f, 0.f, 0.f);

    // The group's rows advance TOGETHER: in every step one nonzero of each row is gathered, so EPB * U
    // independent 16-byte loads per lane are in flight instead of U, and the three dependent latencies of a
    // short row (row pointers, index batch, feature rows) are paid once per packed row, not once per row.
    int64_t e0[EPB];
    int len[EPB];
    int maxlen = 0;
#pragma unroll
    for (int t = 0; t < EPB; ++t) {
        e0[t] = 0, len[t] = 0;
        if (t < cnt) {
            const int lp = long_pos != nullptr ? long_pos[i0 + t] : -1;
            if (lp >= 0) {  // a hub row: summed beforehand by the long-row kernels, many CTAs per row
                const float4 *sp = reinterpret_cast<const float4 *>(long_sums + (int64_t)lp * ld_long);
#pragma unroll
                for (int k = 0; k < NV; ++k)
                    if (gl + GQ * k < FV) acc[t][k] = sp[gl + GQ * k];
            } else {
                e0[t] = rowptr[i0 + t];
                len[t] = (int)(rowptr[i0 + t + 1] - e0[t]);
                maxlen = max(maxlen, len[t]);
            }
        }
    }
    for (int base = 0; base < maxlen; base += GQ) {
        int my_col[EPB];
        float my_val[EPB];
#pragma unroll
        for (int t = 0; t < EPB; ++t) {
            my_col[t] = 0, my_val[t] = 0.f;
            if (base + gl < len[t]) {
                my_col[t] = ld_stream(col + e0[t] + base + gl);
                my_val[t] = ld_stream(val + e0[t] + base + gl);
            }
        }
        const int nb = min(GQ, maxlen - base);
        for (int j0 = 0; j0 < nb; j0 += U) {
            float4 xr[EPB][U][NV];
            float av[EPB][U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = j0 + u;
#pragma unroll
                for (int t = 0; t < EPB; ++t) {
                    const int c = __shfl_sync(gmask, my_col[t], lead + (j & (GQ - 1)));
                    av[t][u] = __shfl_sync(gmask, my_val[t], lead + (j & (GQ - 1)));
                    const float4 *xp = reinterpret_cast<const float4 *>(X + (int64_t)c * ldx);
#pragma unroll
                    for (int k = 0; k < NV; ++k)
                        if (base + j < len[t] && j < nb && gl + GQ * k < FV) xr[t][u][k] = __ldg(xp + gl + GQ * k);
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
#pragma unroll
                for (int t = 0; t < EPB; ++t) {
                    if (base + j0 + u < len[t] && j0 + u < nb) {  // every row keeps its own CSR order
#pragma unroll
                        for (int k = 0; k < NV; ++k)
                            if (gl + GQ * k < FV) {
                                acc[t][k].x = fmaf(av[t][u], xr[t][u][k].x, acc[t][k].x);
                                acc[t][k].y = fmaf(av[t][u], xr[t][u][k].y, acc[t][k].y);
                                acc[t][k].z = fmaf(av[t][u], xr[t][u][k].z, acc[t][k].z);
                                acc[t][k].w = fmaf(av[t][u], xr[t][u][k].w, acc[t][k].w);
                            }
                    }
                }
            }
        }
    }
    quant_pack_group<BITS, NV, GQ>(acc, cnt, i0, R, gl, gmask, lead, FV, F, 0, params, params_bf16, codes);
}

// ---- generic path: any F, any alignment; rows are read twice (second pass hits L1/L2) ----
__global__ void __launch_bounds__(kCodecWarps * 32)
    quant_pack_generic_kernel(const float *__restrict__ X, int64_t ldx, const int32_t *__restrict__ idx, int F,
                              const int32_t *__restrict__ seg, int P, int bits, int params_given,
                              float *__restrict__ params, __nv_bfloat16 *__restrict__ params_bf16,
                              uint8_t *__restrict__ codes) {
    const int epb = 8 / bits;
    const float levels = (float)((1 << bits) - 1);
    __shared__ int pbase[kMaxSeg + 1];
    build_packed_prefix(seg, P, epb, pbase);
    const int lane = threadIdx.x & 31;
    // grid-stride over packed rows: a warp keeps working, so its loads overlap the previous row's stores
    for (int64_t R = (int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5); R < pbase[P];
         R += (int64_t)gridDim.x * kCodecWarps) {
    const int p = find_segment(pbase, P, (int)R);
    const int i0 = seg[p] + ((int)R - pbase[p]) * epb;
    const int cnt = min(epb, seg[p + 1] - i0);

    float zp[8], sc[8];
    const float *xp[8];
#pragma unroll
    for (int t = 0; t < 8; ++t) {
        zp[t] = 0.f, sc[t] = 1.f, xp[t] = X;
        if (t < cnt) {
            const int64_t src = idx ? (int64_t)idx[i0 + t] : (int64_t)(i0 + t);
            xp[t] = X + src * ldx;
            if (!params_given) {
                float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
                int zkey = INT_MAX;
                for (int k = lane; k < F; k += 32) {
                    const float e = xp[t][k];
                    mn = fminf(mn, e), mx = fmaxf(mx, e);
                    if (e == 0.0f && zkey == INT_MAX) zkey = (k << 1) | (int)(__float_as_uint(e) >> 31);
                }
                mn = warp_min(mn), mx = warp_max(mx);
                const float x0 = xp[t][0];
                mn = fix_extreme(mn, x0, zkey);
                mx = fix_extreme(mx, x0, zkey);
                float s = __fdiv_rn(__fsub_rn(mx, mn), levels);
                if (s == 0.0f) s = 1.0f;
                zp[t] = mn, sc[t] = s;
                if (lane == 0) {
                    params[(int64_t)(i0 + t) * 2] = mn;
                    params[(int64_t)(i0 + t) * 2 + 1] = s;
                }
            } else {
                zp[t] = params[(int64_t)(i0 + t) * 2];
                sc[t] = params[(int64_t)(i0 + t) * 2 + 1];
            }
            if (lane == 0 && params_bf16) {
                params_bf16[(int64_t)(i0 + t) * 2] = __float2bfloat16_rn(zp[t]);
                params_bf16[(int64_t)(i0 + t) * 2 + 1] = __float2bfloat16_rn(sc[t]);
            }
        }
    }
    uint8_t *out = codes + R * (int64_t)F;
    for (int k = lane; k < F; k += 32) {
        uint32_t b = 0;
#pragma unroll
        for (int t = 0; t < 8; ++t)
            if (t < cnt) b |= encode(xp[t][k], zp[t], sc[t], params_given) << ((epb - 1 - t) * bits);
        out[k] = (uint8_t)b;
    }
    }  // packed rows
}

// ---- unpack + dequantise -----------------------------------------------------------------
template <int BITS, bool VEC>
__global__ void __launch_bounds__(kCodecWarps * 32)
    unpack_dequant_kernel(const uint8_t *__restrict__ codes, int F, const int32_t *__restrict__ seg, int P,
                          float *__restrict__ params, const __nv_bfloat16 *__restrict__ params_bf16,
                          float *__restrict__ OUT, int64_t ldo) {
    constexpr int EPB = 8 / BITS;
    constexpr uint32_t MASK = (1u << BITS) - 1u;
    __shared__ int pbase[kMaxSeg + 1];
    build_packed_prefix(seg, P, EPB, pbase);
    const int lane = threadIdx.x & 31;
    // grid-stride over packed rows: a warp keeps working, so its loads overlap the previous row's stores
    for (int64_t R = (int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5); R < pbase[P];
         R += (int64_t)gridDim.x * kCodecWarps) {
    const int p = find_segment(pbase, P, (int)R);
    const int i0 = seg[p] + ((int)R - pbase[p]) * EPB;
    const int cnt = min(EPB, seg[p + 1] - i0);

    float zp[EPB], sc[EPB];
#pragma unroll
    for (int t = 0; t < EPB; ++t) {
        zp[t] = 0.f, sc[t] = 0.f;
        if (t < cnt) {
            if (params_bf16) {
                zp[t] = __bfloat162float(params_bf16[(int64_t)(i0 + t) * 2]);
                sc[t] = __bfloat162float(params_bf16[(int64_t)(i0 + t) * 2 + 1]);
                if (params && lane == 0) {
                    params[(int64_t)(i0 + t) * 2] = zp[t];
                    params[(int64_t)(i0 + t) * 2 + 1] = sc[t];
                }
            } else {
                zp[t] = params[(int64_t)(i0 + t) * 2];
                sc[t] = params[(int64_t)(i0 + t) * 2 + 1];
            }
        }
    }
    const uint8_t *in = codes + R * (int64_t)F;
    if (VEC) {
        const uint32_t *in4 = reinterpret_cast<const uint32_t *>(in);
        for (int vi = lane; vi < (F >> 2); vi += 32) {
            const uint32_t w = __ldcs(in4 + vi);
#pragma unroll
            for (int t = 0; t < EPB; ++t) {
                if (t < cnt) {
                    const int sh = (EPB - 1 - t) * BITS;
                    float4 o;
                    o.x = fmaf((float)((w >> sh) & MASK), sc[t], zp[t]);
                    o.y = fmaf((float)((w >> (8 + sh)) & MASK), sc[t], zp[t]);
                    o.z = fmaf((float)((w >> (16 + sh)) & MASK), sc[t], zp[t]);
                    o.w = fmaf((float)((w >> (24 + sh)) & MASK), sc[t], zp[t]);
                    *(reinterpret_cast<float4 *>(OUT + (int64_t)(i0 + t) * ldo) + vi) = o;
                }
            }
        }
    } else {
        for (int k = lane; k < F; k += 32) {
            const uint32_t w = in[k];
#pragma unroll
            for (int t = 0; t < EPB; ++t)
                if (t < cnt)
                    OUT[(int64_t)(i0 + t) * ldo + k] = fmaf((float)((w >> ((EPB - 1 - t) * BITS)) & MASK), sc[t], zp[t]);
        }
    }
    }  // packed rows
}

// ---- mixed-bit column-packed codec: one warp per row ------------------------------------
__global__ void __launch_bounds__(kCodecWarps * 32)
    quant_v1_kernel(const float *__restrict__ X, int64_t ldx, int64_t rows, int F, const int64_t *__restrict__ range,
                    float *__restrict__ params, uint8_t *__restrict__ codes) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5);
    if (i >= rows) return;
    const float *xp = X + i * ldx;
    const int bits = (int)params[i * 3];
    if (bits != 8 && bits != 4 && bits != 2) return;  // the reference prints an error and skips the row
    float mn = __int_as_float(0x7f800000), mx = __int_as_float(0xff800000);
    int zkey = INT_MAX;
    for (int k = lane; k < F; k += 32) {
        const float e = xp[k];
        mn = fminf(mn, e), mx = fmaxf(mx, e);
        if (e == 0.0f && zkey == INT_MAX) zkey = (k << 1) | (int)(__float_as_uint(e) >> 31);
    }
    mn = warp_min(mn), mx = warp_max(mx);
    const float x0 = xp[0];
    mn = fix_extreme(mn, x0, zkey);
    mx = fix_extreme(mx, x0, zkey);
    float s = __fdiv_rn(__fsub_rn(mx, mn), (float)((1 << bits) - 1));
    if (s == 0.0f) s = 1.0f;
    if (lane == 0) {
        params[i * 3 + 1] = mn;
        params[i * 3 + 2] = s;
    }
    const int epb = 8 / bits;
    uint8_t *out = codes + range[i];
    const int nbytes = (F + epb - 1) / epb;
    for (int j = lane; j < nbytes; j += 32) {
        uint32_t b = 0;
        for (int k = 0; k < epb && j * epb + k < F; ++k)
            b |= ((uint32_t)__float2int_rn(__fdiv_rn(__fsub_rn(xp[j * epb + k], mn), s))) << ((epb - 1 - k) * bits);
        out[j] = (uint8_t)b;
    }
}

__global__ void __launch_bounds__(kCodecWarps * 32)
    dequant_v1_kernel(const uint8_t *__restrict__ codes, int64_t rows, int F, const int64_t *__restrict__ range,
                      const float *__restrict__ params, float *__restrict__ OUT, int64_t ldo) {
    const int lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * kCodecWarps + (threadIdx.x >> 5);
    if (i >= rows) return;
    const int bits = (int)params[i * 3];
    if (bits != 8 && bits != 4 && bits != 2) return;
    const float zp = params[i * 3 + 1], s = params[i * 3 + 2];
    const int epb = 8 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    const uint8_t *in = codes + range[i];
    const int64_t plen = range[i + 1] - range[i];
    for (int k = lane; k < F; k += 32) {
        const int j = k / epb;
        if (j < plen) {
            const uint32_t b = in[j];
            // val*scale + zp: one fma under the reference's build flags (GCC contracts it)
            OUT[i * ldo + k] = fmaf((float)((b >> ((epb - 1 - (k % epb)) * bits)) & mask), s, zp);
        }
    }
}

}  // namespace gnnagg

using namespace gnnagg;

static int check_seg_args(const char *who, const int32_t *seg, int32_t P, int64_t rows, int32_t bits, int32_t F) {
    if (seg == nullptr || P < 1 || rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "%s: bad seg / P / rows / F", who);
    if (bits != 2 && bits != 4 && bits != 8) return fail(GNNAGG_ERR_ARG, "%s: bits must be 2, 4 or 8", who);
    if (P > kMaxSeg) return fail(GNNAGG_ERR_UNSUPPORTED, "%s: more than %d segments", who, kMaxSeg);
    if (rows > INT32_MAX) return fail(GNNAGG_ERR_UNSUPPORTED, "%s: rows must fit int32", who);
    return GNNAGG_OK;
}

// Upper bound of the number of packed rows: the exact count lives on the device (seg), the
// launch only needs a grid that covers it.
static int64_t packed_rows_bound(int64_t rows, int32_t P, int epb) { return div_up(rows, epb) + P; }

// CTAs for the grid-stride codec kernels: enough to cover the rows, at most 16 per SM.
static unsigned codec_blocks(int64_t rows, int32_t P, int epb) {
    int64_t b = div_up(packed_rows_bound(rows, P, epb), kCodecWarps);
    const int64_t cap = (int64_t)kNumSMs * 32;
    return (unsigned)(b < cap ? b : cap);
}

extern "C" int gnnagg_quant_pack_rows(const float *X, int64_t ldx, const int32_t *idx, int32_t F, const int32_t *seg,
                                      int32_t P, int64_t rows, int32_t bits, int32_t params_given, float *params,
                                      void *params_bf16, uint8_t *codes, void *stream) {
    int rc = check_seg_args("quant_pack_rows", seg, P, rows, bits, F);
    if (rc != GNNAGG_OK) return rc;
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (X == nullptr || params == nullptr || codes == nullptr || ldx < F)
        return fail(GNNAGG_ERR_ARG, "quant_pack_rows: null pointer or ldx < F");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int epb = 8 / bits;
    const unsigned blocks = codec_blocks(rows, P, epb);
    const bool vec = (F % 4 == 0) && (ldx % 4 == 0) && aligned16(X) && F <= 512 &&
                     (reinterpret_cast<uintptr_t>(codes) % 4 == 0) && (reinterpret_cast<uintptr_t>(params) % 8 == 0) &&
                     (params_bf16 == nullptr || reinterpret_cast<uintptr_t>(params_bf16) % 4 == 0);
    if (vec) {
        uint32_t *pb = static_cast<uint32_t *>(params_bf16);
#define GNNAGG_QP(B, NV, GQ)                                                                                      \
    quant_pack_vec_kernel<B, NV, GQ><<<blocks, kCodecWarps * 32, 0, st>>>(X, ldx, idx, F, seg, P, params_given, params, \
                                                                           pb, codes)
#define GNNAGG_QP_WIDTH(B)                                         \
    do {                                                           \
        if (F <= 32) GNNAGG_QP(B, 1, 8);                           \
        else if (F <= 64) GNNAGG_QP(B, 1, 16);                     \
        else if (F <= 128) GNNAGG_QP(B, 1, 32);                    \
        else if (F <= 256) GNNAGG_QP(B, 2, 32);                    \
        else GNNAGG_QP(B, 4, 32);                                  \
    } while (0)
        if (bits == 2) GNNAGG_QP_WIDTH(2);
        else if (bits == 4) GNNAGG_QP_WIDTH(4);
        else GNNAGG_QP_WIDTH(8);
#undef GNNAGG_QP_WIDTH
#undef GNNAGG_QP
        return check_launch("quant_pack_vec_kernel");
    }
    quant_pack_generic_kernel<<<blocks, kCodecWarps * 32, 0, st>>>(X, ldx, idx, F, seg, P, bits, params_given, params,
                                                                  static_cast<__nv_bfloat16 *>(params_bf16), codes);
    return check_launch("quant_pack_generic_kernel");
}

// Gather steps issued back to back by the fused SpMM + pack kernel: 8 / bits rows advance together, so
// rows * steps * NV 16-byte loads are in flight per lane -- eight, or sixteen for 2-bit codes on rows of
// more than 128 floats, where one step alone would leave the memory system idle.
static constexpr int sq_steps(int bits, int nv) {
    const int rows = 8 / bits;
    const int u = 8 / (rows * nv);
    return (rows == 4 && nv == 2) ? 2 : (u < 1 ? 1 : u);
}

extern "C" int gnnagg_spmm_quant_pack(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                                      int64_t nnz, const float *X, int64_t ldx, int32_t F, const int32_t *seg,
                                      int32_t P, int32_t bits, const int32_t *long_pos, const float *long_sums,
                                      int64_t ld_long, float *params, void *params_bf16, uint8_t *codes,
                                      void *stream) {
    int rc = check_seg_args("spmm_quant_pack", seg, P, M, bits, F);
    if (long_pos != nullptr && (long_sums == nullptr || ld_long < F || ld_long % 4 != 0 || !aligned16(long_sums)))
        return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: long-row sums missing, misaligned or narrower than F");
    if (rc != GNNAGG_OK) return rc;
    if (K < 0 || nnz < 0) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: negative size");
    if (M == 0 || F == 0) return GNNAGG_OK;
    if (rowptr == nullptr || params == nullptr || codes == nullptr || (nnz > 0 && (col == nullptr || val == nullptr || X == nullptr)))
        return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: null pointer");
    if (ldx < F) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: ldx < F");
    const bool ok = (F % 4 == 0) && F <= 512 && (ldx % 4 == 0) && aligned16(X) &&
                    (reinterpret_cast<uintptr_t>(codes) % 4 == 0) && (reinterpret_cast<uintptr_t>(params) % 8 == 0) &&
                    (params_bf16 == nullptr || reinterpret_cast<uintptr_t>(params_bf16) % 4 == 0);
    if (!ok)
        return fail(GNNAGG_ERR_UNSUPPORTED,
                    "spmm_quant_pack: needs F %% 4 == 0, F <= 512 and 16-byte aligned dense rows; use gnnagg_spmm_csr_f32 "
                    "followed by gnnagg_quant_pack_rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int epb = 8 / bits;
    uint32_t *pb = static_cast<uint32_t *>(params_bf16);
    const int64_t groups = packed_rows_bound(M, P, epb);
#define GNNAGG_SQ(B, NV, GQ, U)                                                                                        \
    spmm_quant_pack_kernel<B, NV, GQ, U><<<(unsigned)div_up(groups, kCodecWarps * (32 / GQ)), kCodecWarps * 32, 0, st>>>( \
        rowptr, col, val, X, ldx, F, seg, P, long_pos, long_sums, ld_long, params, pb, codes)
#define GNNAGG_SQ_WIDTH(B)                                       \
    do {                                                         \
        if (F <= 32) GNNAGG_SQ(B, 1, 8, sq_steps(B, 1));           \
        else if (F <= 64) GNNAGG_SQ(B, 1, 16, sq_steps(B, 1));     \
        else if (F <= 128) GNNAGG_SQ(B, 1, 32, sq_steps(B, 1));    \
        else if (F <= 256) GNNAGG_SQ(B, 2, 32, sq_steps(B, 2));    \
        else GNNAGG_SQ(B, 4, 32, sq_steps(B, 4));                  \
    } while (0)
    if (bits == 2) GNNAGG_SQ_WIDTH(2);
    else if (bits == 4) GNNAGG_SQ_WIDTH(4);
    else GNNAGG_SQ_WIDTH(8);
#undef GNNAGG_SQ_WIDTH
#undef GNNAGG_SQ
    return check_launch("spmm_quant_pack_kernel");
}

extern "C" int32_t gnnagg_spmm_long_row_threshold(void) { return kLongSeg / 8; }
extern "C" int32_t gnnagg_spmm_long_row_segment(void) { return kLongSeg; }

extern "C" int gnnagg_spmm_long_rows(const int64_t *rowptr, const int32_t *col, const float *val, const float *X,
                                     int64_t ldx, int32_t F, const int32_t *long_idx, int32_t L,
                                     const int32_t *seg_row, const int32_t *seg_off, const int32_t *row_seg_ptr,
                                     int32_t S, float *partial, float *sums, int64_t ld, void *stream) {
    if (L < 0 || S < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "spmm_long_rows: negative size");
    if (L == 0 || S == 0 || F == 0) return GNNAGG_OK;
    if (rowptr == nullptr || col == nullptr || val == nullptr || X == nullptr || long_idx == nullptr || seg_row == nullptr ||
        seg_off == nullptr || row_seg_ptr == nullptr || partial == nullptr || sums == nullptr)
        return fail(GNNAGG_ERR_ARG, "spmm_long_rows: null pointer");
    if (F % 4 != 0 || F > 512 || ldx % 4 != 0 || ld % 4 != 0 || ld < F || !aligned16(X) || !aligned16(partial) || !aligned16(sums))
        return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_long_rows: needs F %% 4 == 0, F <= 512 and 16-byte aligned rows");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int FV = F / 4;
#define GNNAGG_LR(NV, U) \
    spmm_long_rows_partial_kernel<NV, U><<<(unsigned)S, 128, 0, st>>>(rowptr, col, val, X, ldx, FV, long_idx, seg_row, seg_off, partial, ld)
    if (F <= 128) GNNAGG_LR(1, 8);
    else if (F <= 256) GNNAGG_LR(2, 4);
    else GNNAGG_LR(4, 2);
#undef GNNAGG_LR
    int rc = check_launch("spmm_long_rows_partial_kernel");
    if (rc != GNNAGG_OK) return rc;
    spmm_long_rows_reduce_kernel<<<(unsigned)L, 128, 0, st>>>(row_seg_ptr, L, partial, sums, ld, F);
    return check_launch("spmm_long_rows_reduce_kernel");
}

extern "C" int gnnagg_unpack_dequant_rows(const uint8_t *codes, int32_t F, const int32_t *seg, int32_t P, int64_t rows,
                                          int32_t bits, float *params, const void *params_bf16, float *OUT,
                                          int64_t ldo, void *stream) {
    int rc = check_seg_args("unpack_dequant_rows", seg, P, rows, bits, F);
    if (rc != GNNAGG_OK) return rc;
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (codes == nullptr || OUT == nullptr || (params == nullptr && params_bf16 == nullptr) || ldo < F)
        return fail(GNNAGG_ERR_ARG, "unpack_dequant_rows: null pointer or ldo < F");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int epb = 8 / bits;
    const unsigned blocks = codec_blocks(rows, P, epb);
    const __nv_bfloat16 *pb = static_cast<const __nv_bfloat16 *>(params_bf16);
    const bool vec = (F % 4 == 0) && (ldo % 4 == 0) && aligned16(OUT) && (reinterpret_cast<uintptr_t>(codes) % 4 == 0);
#define GNNAGG_UD(B, V) \
    unpack_dequant_kernel<B, V><<<blocks, kCodecWarps * 32, 0, st>>>(codes, F, seg, P, params, pb, OUT, ldo)
    if (bits == 2) {
        if (vec) GNNAGG_UD(2, true); else GNNAGG_UD(2, false);
    } else if (bits == 4) {
        if (vec) GNNAGG_UD(4, true); else GNNAGG_UD(4, false);
    } else {
        if (vec) GNNAGG_UD(8, true); else GNNAGG_UD(8, false);
    }
#undef GNNAGG_UD
    return check_launch("unpack_dequant_kernel");
}

extern "C" int gnnagg_quant_v1_rows(const float *X, int64_t ldx, int64_t rows, int32_t F, const int64_t *range,
                                    float *params, uint8_t *codes, void *stream) {
    if (rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "quant_v1_rows: negative size");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (X == nullptr || range == nullptr || params == nullptr || codes == nullptr || ldx < F)
        return fail(GNNAGG_ERR_ARG, "quant_v1_rows: null pointer or ldx < F");
    quant_v1_kernel<<<(unsigned)div_up(rows, kCodecWarps), kCodecWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        X, ldx, rows, F, range, params, codes);
    return check_launch("quant_v1_kernel");
}

extern "C" int gnnagg_dequant_v1_rows(const uint8_t *codes, int64_t rows, int32_t F, const int64_t *range,
                                      const float *params, float *OUT, int64_t ldo, void *stream) {
    if (rows < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "dequant_v1_rows: negative size");
    if (rows == 0 || F == 0) return GNNAGG_OK;
    if (codes == nullptr || range == nullptr || params == nullptr || OUT == nullptr || ldo < F)
        return fail(GNNAGG_ERR_ARG, "dequant_v1_rows: null pointer or ldo < F");
    dequant_v1_kernel<<<(unsigned)div_up(rows, kCodecWarps), kCodecWarps * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        codes, rows, F, range, params, OUT, ldo);
    return check_launch("dequant_v1_kernel");
}
