/*
 * TEST INFRASTRUCTURE -- CPU oracle for the graph-aggregation hot path.
 *
 * Plain-C restatement of the arithmetic of the reference's native ops
 * (self_benchmark/a64fx/model/ops/src/).  It is the checker the parity tests,
 * the smoke run and the bench's cpu_baseline leg compare the CUDA kernels
 * against.  Nothing in the product package may call into this file.
 *
 * Compile with -ffp-contract=off: every fused multiply-add below is explicit
 * (fmaf) and every other operation must round once per operator, exactly as
 * the vector intrinsics of the reference do.
 *
 * Parity status per function is stated in each header comment:
 *   "pinned"     = checked against a golden vector of the reference's own tests
 *                  or against the reference's compiled x86 module;
 *   "unpinned"   = restated from source only (the ARM SVE int2 kernels cannot be
 *                  compiled on x86 and no reference test holds their bytes).
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

/* ------------------------------------------------------------------------- */
/* SpMM: out[M,F] += A_csr[M,K] * X[K,F]                                      */
/* Follows model/ops/src/spmm.cpp:97-126 (kernel_1xN inner loop) and          */
/* :327-507 (driver): for each row m, for each nonzero e in CSR order,        */
/* out[m,:] = fma(value[e], X[col[e],:], out[m,:]) -- one single-rounded FMA  */
/* per nonzero, accumulating onto what `out` already holds (the kernel loads  */
/* `out` first, :79-95).  The 64-column strips of the reference do not change */
/* any output element: each element is its own sequential FMA chain.          */
/* Pinned: against the compiled reference `spmm` (bit-exact) in               */
/* tests/test_oracle_pins.py when oracle/_ref is built.                       */
/* ------------------------------------------------------------------------- */
void oracle_spmm_csr_f32(const int64_t *rowptr, const int64_t *col, const float *val,
                         int64_t M, const float *X, float *out, int64_t F)
{
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t m = 0; m < M; ++m) {
        float *o = out + m * F;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) {
            const float a = val[e];
            const float *x = X + col[e] * F;
            for (int64_t n = 0; n < F; ++n) o[n] = fmaf(a, x[n], o[n]);
        }
    }
}

/* Same product accumulated in double, for adjudicating fp32 summation-order
 * differences (not part of the reference; an error yardstick only). */
void oracle_spmm_csr_f64acc(const int64_t *rowptr, const int64_t *col, const float *val,
                            int64_t M, const float *X, double *out, int64_t F)
{
#pragma omp parallel for schedule(dynamic, 256)
    for (int64_t m = 0; m < M; ++m) {
        double *o = out + m * F;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) {
            const double a = (double)val[e];
            const float *x = X + col[e] * F;
            for (int64_t n = 0; n < F; ++n) o[n] += a * (double)x[n];
        }
    }
}

/* Greedy nnz-balanced row ranges per thread.
 * Follows model/ops/spmm_kernel.py:7-28 (distribute_work_for_row): the "flops"
 * of a row is the SUM OF ITS VALUES (segment_csr(value, rowptr, "sum")), the
 * target is total // T in float arithmetic of the reference (floor division of
 * fp32 tensors), the running sum restarts at the row that tripped the cut and
 * the cut is placed BEFORE that row.  row_splits has T+1 int32 entries. */
void oracle_distribute_work_for_row(const int64_t *rowptr, const float *val, int64_t M,
                                    int32_t T, int32_t *row_splits)
{
    float *flops = (float *)malloc(sizeof(float) * (size_t)(M > 0 ? M : 1));
    float total = 0.f;
    for (int64_t m = 0; m < M; ++m) {
        float s = 0.f;
        for (int64_t e = rowptr[m]; e < rowptr[m + 1]; ++e) s += val[e];
        flops[m] = s;
    }
    /* torch.sum over fp32 uses pairwise/vectorised summation; for all-ones values
     * (the reference's only use) any order is exact below 2^24 and the split only
     * steers load balance, never results. */
    for (int64_t m = 0; m < M; ++m) total += flops[m];
    const float target = floorf(total / (float)T);
    for (int32_t t = 0; t <= T; ++t) row_splits[t] = (int32_t)M;
    row_splits[0] = 0;
    float cur = 0.f;
    int32_t tid = 0;
    for (int64_t m = 0; m < M; ++m) {
        cur += flops[m];
        if (cur > target && tid < T) {
            row_splits[tid + 1] = (int32_t)m;
            ++tid;
            cur = flops[m];
        }
    }
    row_splits[T] = (int32_t)M;
    free(flops);
}

/* ------------------------------------------------------------------------- */
/* Shared scalar pieces of the quantisers                                     */
/* ------------------------------------------------------------------------- */

/* Row min / max: scan from element 0, replace only on strict > / < so a NaN
 * never replaces and the first of several equal-comparing values (+0 / -0)
 * is kept.  quantization_arm.cpp:93-104, quantization_x86.cpp:189-196
 * (std::max(a,b) is (a<b)?b:a, i.e. the same strict rule). */
static void row_min_max(const float *x, int64_t F, float *mn, float *mx)
{
    float a = x[0], b = x[0];
    for (int64_t k = 1; k < F; ++k) {
        const float v = x[k];
        if (v > b) b = v;
        if (v < a) a = v;
    }
    *mn = a;
    *mx = b;
}

/* float -> unsigned conversion of an already-rounded value with the semantics of
 * the SVE FCVTZU used at quantization_arm.cpp:153-156: NaN -> 0, negatives -> 0,
 * overflow saturates. */
static uint32_t cvt_u32_sat(float r)
{
    if (!(r == r)) return 0u;
    if (r <= 0.f) return 0u;
    if (r >= 4294967296.f) return 0xFFFFFFFFu;
    return (uint32_t)r;
}

/* code = u32(round_ties_even((x - zp) / scale)): subtract, true IEEE divide, round.
 * quantization_arm.cpp:143-156 (svsub, svdiv, svrintn, svcvt). nearbyintf under the
 * default rounding mode is round-half-to-even. */
static uint32_t encode_one(float x, float zp, float scale)
{
    const float d = x - zp;
    const float q = d / scale;
    return cvt_u32_sat(nearbyintf(q));
}

/* ------------------------------------------------------------------------- */
/* int2 row-packed codec with per-peer segments (the live training path)      */
/* quantize_tensor_for_all_procs  quantization_arm.cpp:364-435                */
/* quantize_tensor_kernel         quantization_arm.cpp:80-217                 */
/* divide_work_v1                 quantization_arm.cpp:21-78                  */
/*                                                                            */
/* seg[0..P] = prefix of per-peer row counts.  Inside peer p, local row j     */
/* lands in packed row base_p + j/4 with base_p = sum_{q<p} ceil(n_q/4)       */
/* (:30,:51) at bit position 2*(3 - j%4) (:158-161; tail group :204-214).     */
/* The thread split of divide_work_v1 only ever cuts at multiples of four     */
/* rows counted from a segment start (:55-62), so the grouping below is what  */
/* every thread count produces.  bits is ignored by the reference (BITS=2     */
/* hard-coded, :380-381) and is therefore not a parameter here.               */
/* params is (rows,2) fp32 [zero_point, scale] (:112-113).                    */
/* Parity: UNPINNED by any reference test; cross-checked per segment against  */
/* the reference's compiled x86 generic quantize_tensor (same layout, one     */
/* segment) in tests/test_oracle_pins.py, which is the invariant the          */
/* reference's own tests/test_quantization_ops.py:223-245 prints.             */
/* ------------------------------------------------------------------------- */
void oracle_quantize_int2_for_all_procs(const float *x, int64_t F, const int32_t *seg, int32_t P,
                                        uint8_t *codes, float *params)
{
    int64_t base = 0;
    for (int32_t p = 0; p < P; ++p) {
        const int64_t r0 = seg[p], n = seg[p + 1] - seg[p];
        for (int64_t j = 0; j < n; ++j) {
            const int64_t i = r0 + j;
            float mn, mx;
            row_min_max(x + i * F, F, &mn, &mx);
            float scale = (mx - mn) / (float)((1 << 2) - 1);
            if (scale == 0) scale = 1.0f;
            params[i * 2] = mn;
            params[i * 2 + 1] = scale;
        }
        const int64_t groups = (n + 3) / 4;
        for (int64_t g = 0; g < groups; ++g) {
            uint8_t *out = codes + (base + g) * F;
            const int64_t lanes = (n - g * 4) < 4 ? (n - g * 4) : 4;
            for (int64_t k = 0; k < F; ++k) {
                uint32_t byte = 0;
                for (int64_t t = 0; t < lanes; ++t) {
                    const int64_t i = r0 + g * 4 + t;
                    const uint32_t q = encode_one(x[i * F + k], params[i * 2], params[i * 2 + 1]);
                    byte |= q << (2 * (3 - t));
                }
                out[k] = (uint8_t)byte; /* svst1b keeps the low byte */
            }
        }
        base += groups;
    }
}

/* dequantize_tensor_for_all_procs quantization_arm.cpp:437-479,
 * dequantize_tensor_kernel :219-299: y = fma(float(code), scale, zp) (:262-265, :293). */
void oracle_dequantize_int2_for_all_procs(const uint8_t *codes, int64_t F, const int32_t *seg,
                                          int32_t P, const float *params, float *y)
{
    int64_t base = 0;
    for (int32_t p = 0; p < P; ++p) {
        const int64_t r0 = seg[p], n = seg[p + 1] - seg[p];
        for (int64_t j = 0; j < n; ++j) {
            const int64_t i = r0 + j;
            const uint8_t *in = codes + (base + j / 4) * F;
            const int sh = 2 * (3 - (int)(j % 4));
            const float zp = params[i * 2], sc = params[i * 2 + 1];
            for (int64_t k = 0; k < F; ++k)
                y[i * F + k] = fmaf((float)((in[k] >> sh) & 3u), sc, zp);
        }
        base += (n + 3) / 4;
    }
}

/* ------------------------------------------------------------------------- */
/* Generic row-packed codec, caller-supplied min / scale, bits in {8,4,2}     */
/* quantize_tensor / dequantize_tensor  quantization_x86.cpp:17-168           */
/* 8/bits consecutive rows share a byte per column, first row in the high     */
/* bits (:75, :92).  Rounding: cvt_roundps to nearest-even (:74) / nearbyint  */
/* (:90).  The conversion is to SIGNED int32 there; for in-range inputs the   */
/* results coincide with the unsigned one.  Decode: val*scale + min (:141,     */
/* :154); the reference's build flags (-O3, AVX-512, GCC's default            */
/* -ffp-contract=fast) compile that expression to ONE fused multiply-add,     */
/* which is what fused != 0 evaluates; fused == 0 is the two-rounding reading */
/* of the source.  Pinned: codes and fused decode bit-exact vs the compiled   */
/* module.                                                                    */
/* ------------------------------------------------------------------------- */
void oracle_quantize_rowpacked(const float *x, int64_t rows, int64_t F, const float *mn,
                               const float *scale, int32_t bits, uint8_t *codes)
{
    const int64_t epb = 8 / bits;
    const int64_t groups = (rows + epb - 1) / epb;
    for (int64_t g = 0; g < groups; ++g) {
        const int64_t lanes = (rows - g * epb) < epb ? (rows - g * epb) : epb;
        for (int64_t k = 0; k < F; ++k) {
            uint32_t byte = 0;
            for (int64_t t = 0; t < lanes; ++t) {
                const int64_t i = g * epb + t;
                const float q = nearbyintf((x[i * F + k] - mn[i]) / scale[i]);
                const int32_t v = (int32_t)q;
                byte |= ((uint32_t)v) << ((epb - t - 1) * bits);
            }
            codes[g * F + k] = (uint8_t)byte;
        }
    }
}

void oracle_dequantize_rowpacked(const uint8_t *codes, int64_t rows, int64_t F, const float *mn,
                                 const float *scale, int32_t bits, float *y, int32_t fused)
{
    const int64_t epb = 8 / bits;
    const uint32_t mask = (1u << bits) - 1u;
    for (int64_t i = 0; i < rows; ++i) {
        const int sh = (int)((epb - (i % epb) - 1) * bits);
        const uint8_t *in = codes + (i / epb) * F;
        for (int64_t k = 0; k < F; ++k) {
            const float v = (float)((in[k] >> sh) & mask);
            if (fused) {
                y[i * F + k] = fmaf(v, scale[i], mn[i]);
            } else {
                const float m = v * scale[i];
                y[i * F + k] = m + mn[i];
            }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Mixed-bit column-packed codec (per-row bits 8/4/2)                         */
/* quantize_tensor_v1 / dequantize_tensor_v1  quantization_x86.cpp:170-312,   */
/* quantization_arm.cpp:481-603; 8-bit rows via quantization_kernel_x86.h:    */
/* 11-75.  params (rows,3) fp32 [bits, zp, scale]; bits is read from          */
/* params[i,0] (:201), scale = (max-min)/(2^bits-1), 0 -> 1 (:203-205); row i */
/* occupies bytes [range[i], range[i+1]); element k goes to byte k/epb,       */
/* shifted left by bits*(epb-1-k%epb) (:242); decode val*scale+zp (:301).     */
/* Pinned: golden bytes of the reference's tests/test_quantizer.py:57-84 and  */
/* bit-exact vs the compiled module.                                          */
/* ------------------------------------------------------------------------- */
void oracle_quantize_v1(const float *x, int64_t rows, int64_t F, const int64_t *range,
                        float *params, uint8_t *codes)
{
    for (int64_t i = 0; i < rows; ++i) {
        float mn, mx;
        row_min_max(x + i * F, F, &mn, &mx);
        const int bits = (int)params[i * 3];
        float scale = (mx - mn) / (float)((1 << bits) - 1);
        if (scale == 0) scale = 1.0f;
        params[i * 3 + 1] = mn;
        params[i * 3 + 2] = scale;
        const int64_t epb = 8 / bits;
        for (int64_t j = 0; j < F; j += epb) {
            const int64_t rem = (F - j) < epb ? (F - j) : epb;
            uint32_t byte = 0;
            for (int64_t k = 0; k < rem; ++k) {
                const int32_t v = (int32_t)lrintf((x[i * F + j + k] - mn) / scale);
                byte |= ((uint32_t)v) << ((epb - k - 1) * bits);
            }
            codes[range[i] + j / epb] = (uint8_t)byte;
        }
    }
}

/* fused != 0 evaluates the decode as one fma -- what the reference's own build flags
 * produce (GCC contracts val*scale+zp; verified bit-exact against the compiled
 * module) -- 0 as multiply then add (the source read literally). */
void oracle_dequantize_v1(const uint8_t *codes, int64_t rows, int64_t F, const int64_t *range,
                          const float *params, float *y, int32_t fused)
{
    for (int64_t i = 0; i < rows; ++i) {
        const int bits = (int)params[i * 3];
        const float zp = params[i * 3 + 1], scale = params[i * 3 + 2];
        const int64_t epb = 8 / bits;
        const uint32_t mask = (1u << bits) - 1u;
        const int64_t plen = range[i + 1] - range[i];
        for (int64_t j = 0; j < plen; ++j) {
            const uint8_t b = codes[range[i] + j];
            for (int64_t k = 0; k < epb && j * epb + k < F; ++k) {
                const float v = (float)((b >> ((epb - k - 1) * bits)) & mask);
                float r;
                if (fused) {
                    r = fmaf(v, scale, zp);
                } else {
                    const float m = v * scale;
                    r = m + zp;
                }
                y[i * F + j * epb + k] = r;
            }
        }
    }
}

/* fp32 -> bf16 -> fp32 with round-to-nearest-even, the wire format of the
 * quantisation parameters (communicator.py:297-303: Tensor.copy_ between fp32
 * and bfloat16 buffers).  NaN stays NaN (quiet). */
void oracle_bf16_round(const float *x, int64_t n, float *y)
{
    for (int64_t i = 0; i < n; ++i) {
        uint32_t u;
        memcpy(&u, &x[i], 4);
        if ((u & 0x7F800000u) == 0x7F800000u && (u & 0x007FFFFFu)) {
            u = (u | 0x00400000u) & 0xFFFF0000u;
        } else {
            const uint32_t lsb = (u >> 16) & 1u;
            u += 0x7FFFu + lsb;
            u &= 0xFFFF0000u;
        }
        memcpy(&y[i], &u, 4);
    }
}

int oracle_num_threads(void)
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
