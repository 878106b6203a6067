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
#include "codec.cuh"

namespace gnnagg {

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
