// K1: merge-path CSR SpMM for sm_100a,  Y[M,F] (+)= A[M,K] * X[K,F], fp32.
//
// Work decomposition (the "plan", built once per sparsity pattern):
//   the M row-end events and the nnz nonzeros are merged into one list of M+nnz items
//   (merge-path); the list is cut every kItems items and one WARP owns one chunk.  A cut
//   that lands inside a row no longer than a chunk is moved forward to the end of that
//   row, so only hub rows (longer than a chunk) are ever shared between warps.
// Per chunk a warp
//   - streams its slice of col/val into shared memory with asynchronous copies, one 256-nonzero
//     tile ahead of its use, and reads every nonzero from there with a broadcast load,
//   - gathers feature rows with 128-bit loads: G = min(32, F/4 rounded up to a power of
//     two) lanes cover one feature row, so S = 32/G nonzeros are fetched per warp load
//     instruction and U such instructions are issued back to back before any is consumed
//     (U*NV independent 16-byte loads in flight per lane),
//   - applies one fused multiply-add per nonzero in CSR order (the reference's order,
//     model/ops/src/spmm.cpp:97-126); when accumulating, the chain starts from the old
//     output row (fetched one row ahead), exactly as the reference loads `out` first
//     (spmm.cpp:79-95); at every row end it folds the S lane groups with xor-shuffles and
//     writes the row once with streaming stores.
// A row cut across chunks is finished by the chunk that holds its row end; the earlier
// chunks park their partial sums in `scratch` and a second small kernel adds them in chunk
// order -- deterministic, no float atomics.
//
// HBM traffic per launch: nnz*(4+4) index/value bytes + one 4F-byte gather per nonzero
// (less what L2 catches) + (M+1)*8 rowptr + M*F*4 output (+ the same again when
// accumulating).
#include <limits.h>

#include "codec.cuh"

namespace gnnagg {

// Launch shape, measured on B200 with the R-MAT scale-22 benchmark matrix: 64-thread CTAs; kernels
// with one vector per lane (F <= 128) run best capped at 85 registers (24 warps per SM resident),
// the wider ones (two to four vectors per lane, more gathers in flight per lane) uncapped.
#ifndef GNNAGG_SPMM_WARPS
#define GNNAGG_SPMM_WARPS 2
#endif
#ifndef GNNAGG_SPMM_MINBLOCKS_NARROW
#define GNNAGG_SPMM_MINBLOCKS_NARROW 12
#endif
#ifndef GNNAGG_SPMM_MINBLOCKS_WIDE
#define GNNAGG_SPMM_MINBLOCKS_WIDE 8
#endif
constexpr int kWarpsPerBlock = GNNAGG_SPMM_WARPS;
// register cap per thread = 65536 / (threads per CTA * min CTAs per SM)
constexpr int min_blocks_per_sm(int nv) { return nv == 1 ? GNNAGG_SPMM_MINBLOCKS_NARROW : GNNAGG_SPMM_MINBLOCKS_WIDE; }
// nonzeros of a chunk are staged through shared memory in tiles of this many (two tiles per warp, the next
// one in flight while the current one is consumed)
constexpr int kTile = 256;
constexpr uint32_t kPlanMagic = 0x4d50534eu;  // "NSPM"
constexpr int kDefaultItems = 512;

struct PlanHeader {
    uint32_t magic;
    int32_t items;
    int64_t M;
    int64_t nnz;
    int64_t nchunks;
    int64_t pad[4];
};
static_assert(sizeof(PlanHeader) == 64, "plan header is 64 bytes");

static int chunk_items() { return kDefaultItems; }

static int64_t num_chunks(int64_t M, int64_t nnz, int items) {
    const int64_t n = div_up(M + nnz, items);
    return n > 0 ? n : 1;
}

static const int64_t *plan_chunk_nz(const void *plan) {
    return reinterpret_cast<const int64_t *>(static_cast<const char *>(plan) + sizeof(PlanHeader));
}
static const int32_t *plan_chunk_row(const void *plan, int64_t nchunks) { return reinterpret_cast<const int32_t *>(plan_chunk_nz(plan) + (nchunks + 1)); }

// One thread per chunk boundary: merge-path diagonal search, then snap to a row end.
__global__ void spmm_plan_kernel(const int64_t *__restrict__ rowptr, int64_t M, int64_t nnz, int items,
                                 int64_t nchunks, PlanHeader *hdr, int64_t *__restrict__ chunk_nz,
                                 int32_t *__restrict__ chunk_row) {
    const int64_t c = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (c == 0) {
        hdr->magic = kPlanMagic;
        hdr->items = items;
        hdr->M = M;
        hdr->nnz = nnz;
        hdr->nchunks = nchunks;
    }
    if (c > nchunks) return;
    int64_t diag = c * (int64_t)items;
    if (diag > M + nnz || c == nchunks) diag = M + nnz;
    int64_t lo = diag > nnz ? diag - nnz : 0;
    int64_t hi = diag < M ? diag : M;
    while (lo < hi) {
        const int64_t mid = (lo + hi) >> 1;
        // row-end event of row `mid` precedes nonzero number (diag-1-mid)?
        if (rowptr[mid + 1] <= diag - 1 - mid)
            lo = mid + 1;
        else
            hi = mid;
    }
    int64_t r = lo, e = diag - lo;
    if (r < M) {
        const int64_t rs = rowptr[r], re = rowptr[r + 1];
        if (e > rs && re - rs <= items) {  // inside a short row: give the whole row to the earlier chunk
            e = re;
            r = r + 1;
        }
    }
    chunk_nz[c] = e;
    chunk_row[c] = (int32_t)r;
}

template <int VW>
struct Vec {
    float v[VW];
};

template <int VW>
__device__ __forceinline__ Vec<VW> vload(const float *p);
template <>
__device__ __forceinline__ Vec<4> vload<4>(const float *p) {
    const float4 t = ld_nc_v4(p);
    Vec<4> r;
    r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
    return r;
}
template <>
__device__ __forceinline__ Vec<1> vload<1>(const float *p) {
    Vec<1> r;
    r.v[0] = ld_nc(p);
    return r;
}
template <int VW>
__device__ __forceinline__ Vec<VW> vload_plain(const float *p);
template <>
__device__ __forceinline__ Vec<4> vload_plain<4>(const float *p) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    Vec<4> r;
    r.v[0] = t.x, r.v[1] = t.y, r.v[2] = t.z, r.v[3] = t.w;
    return r;
}
template <>
__device__ __forceinline__ Vec<1> vload_plain<1>(const float *p) {
    Vec<1> r;
    r.v[0] = *p;
    return r;
}
template <int VW>
__device__ __forceinline__ void vstore_stream(float *p, const Vec<VW> &a);
template <>
__device__ __forceinline__ void vstore_stream<4>(float *p, const Vec<4> &a) {
    st_stream_v4(p, make_float4(a.v[0], a.v[1], a.v[2], a.v[3]));
}
template <>
__device__ __forceinline__ void vstore_stream<1>(float *p, const Vec<1> &a) {
    st_stream(p, a.v[0]);
}
template <int VW>
__device__ __forceinline__ void vstore_plain(float *p, const Vec<VW> &a);
template <>
__device__ __forceinline__ void vstore_plain<4>(float *p, const Vec<4> &a) {
    *reinterpret_cast<float4 *>(p) = make_float4(a.v[0], a.v[1], a.v[2], a.v[3]);
}
template <>
__device__ __forceinline__ void vstore_plain<1>(float *p, const Vec<1> &a) {
    *p = a.v[0];
}

// G lanes per feature row, NV vectors of VW floats per lane, U gather instructions in flight.
// ACC: accumulate onto the old output.  FULL: the row is exactly G*NV vectors wide, so no lane
// holds a vector past the row's end and the per-vector predicates vanish.
// QB: 0 = the dense operand is the fp32 matrix X; 2 / 4 / 8 = the dense operand is a row-packed
// quantised halo buffer (codes + bf16 parameters per wire slot, per-peer segments `seg`): column
// index c is a wire slot, its row is decoded on the fly as fma(code, scale, zero_point) -- the
// value the unpack kernel would have written -- and used in the same FMA chain.
struct PackedOperand {
    const uint8_t *codes;     // (sum_p ceil(n_p / (8/QB)), F) bytes, row stride F
    const uint32_t *params;   // per slot: bf16 zero_point (low half), bf16 scale (high half)
    const int32_t *seg;       // P+1 prefix of per-peer slot counts
    int P;
    int F;
};

// PK: 0 = rows are written to Y; 2 / 4 / 8 = rows are quantised + packed as soon as they are summed and Y
// is never touched (the send side of a packed exchange).  A row that lies inside one chunk is encoded
// from the registers that hold its sum; the tail of a row that began in an earlier chunk is parked in
// `pk.head` and the fix-up kernel encodes the row after adding the parked pieces.
struct PackOut {
    uint8_t *codes;         // zero-filled (sum_p ceil(n_p / (8/PK)), F) bytes
    float *params;          // (M, 2) fp32 [zero_point, scale]
    uint32_t *params_bf16;  // optional (M) bf16 pairs
    const int32_t *seg;     // P+1 prefix of per-peer row counts
    int P;
    int F;
    float *head;            // per chunk: the partial sum of its first row when that row began earlier
};

// The encoder is a few hundred instructions; inlined at every place a row can end it would push the gather
// loop out of the instruction cache (measured: warps stalled on instruction fetch 15x more often than on
// anything else).  One out-of-line copy per kernel, called once per row.
template <int BITS, int NV, int G>
__device__ __noinline__ void encode_row(const float4 (&xv)[1][NV], int row, int gl, int FV, int F, float *params,
                                        uint32_t *params_bf16, int sh, uint32_t (&w)[NV]) {
    const unsigned gmask = G == 32 ? kFullMask : ((1u << G) - 1u);
    quant_pack_group<BITS, NV, G, 1>(xv, 1, row, 0, gl, gmask, 0, FV, F, 0, params, params_bf16, nullptr, sh, w);
}

template <int G, int NV, int VW, int U, bool ACC, bool FULL, int QB, int PK>
__global__ void __launch_bounds__(kWarpsPerBlock * 32, (PK ? GNNAGG_SPMM_MINBLOCKS_WIDE : min_blocks_per_sm(NV)))
    spmm_chunk_kernel(const int64_t *__restrict__ rowptr, const int32_t *__restrict__ col,
                      const float *__restrict__ val, int64_t M, const float *__restrict__ X, int64_t ldx,
                      float *__restrict__ Y, int64_t ldy, int FV,
                      const int64_t *__restrict__ chunk_nz, const int32_t *__restrict__ chunk_row, int64_t nchunks,
                      float *__restrict__ carry, int carry_ld, PackedOperand q, PackOut pk) {
    constexpr int S = 32 / G;  // nonzeros fetched per warp-wide gather instruction
    constexpr int EPB = QB ? 8 / QB : 1;
    constexpr int SEGCAP = (QB || PK) ? kMaxSeg + 1 : 1;
    static_assert(!(QB && PK), "a packed operand and a packed result are separate launches");
    __shared__ int sseg[SEGCAP];
    __shared__ int pbase[SEGCAP];
    __shared__ int s_col[kWarpsPerBlock][2][kTile];
    __shared__ float s_val[kWarpsPerBlock][2][kTile];
    __shared__ uint32_t s_prm[QB ? kWarpsPerBlock : 1][2][QB ? kTile : 1];
    if (QB) build_packed_prefix(q.seg, q.P, EPB, pbase, sseg);  // before any warp leaves: it synchronises the CTA
    if (PK) build_packed_prefix(pk.seg, pk.P, 8 / (PK ? PK : 8), pbase, sseg);
    const int lane = threadIdx.x & 31;
    const int wib = threadIdx.x >> 5;
    const int64_t c = (int64_t)blockIdx.x * kWarpsPerBlock + wib;
    if (c >= nchunks) return;
    const int gl = lane % G, grp = lane / G;

    const int64_t e0 = chunk_nz[c], e1 = chunk_nz[c + 1];
    int r = chunk_row[c];
    const int r1 = chunk_row[c + 1];
    const int n = (int)(e1 - e0);

    // Column indices and values of the chunk travel global -> shared asynchronously, a tile ahead of their
    // use; every gather step then reads its nonzero with a broadcast shared-memory load.
    const int ntiles = (n + kTile - 1) / kTile;
    auto issue_tile = [&](int k) {
        const int base = k * kTile;
        const int cnt = (n - base) < kTile ? (n - base) : kTile;
        int *dc = s_col[wib][k & 1];
        float *dv = s_val[wib][k & 1];
        for (int i = lane; i < cnt; i += 32) {
            cp_async_4(dc + i, col + e0 + base + i);
            cp_async_4(dv + i, val + e0 + base + i);
        }
        cp_async_commit();
    };
    if (ntiles > 0) issue_tile(0);

    int voff[NV];
    bool vok[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) {
        voff[k] = (gl + k * G) * VW;
        vok[k] = FULL || (gl + k * G) < FV;
    }

    constexpr bool acc_mode = ACC;
    Vec<VW> acc[NV];    // running sum of the current row (lane group 0 starts from the old Y when accumulating)
    Vec<VW> ynext[NV];  // accumulate mode: old Y of the row after the current one, fetched one row ahead

    // Old output row `row` into dst (lane group 0; zeros elsewhere and when not accumulating).
    auto load_y = [&](int row, Vec<VW>(&dst)[NV]) {
#pragma unroll
        for (int k = 0; k < NV; ++k) {
            if (acc_mode && grp == 0 && vok[k] && row < M) {
                dst[k] = vload_plain<VW>(Y + (int64_t)row * ldy + voff[k]);
            } else {
#pragma unroll
                for (int i = 0; i < VW; ++i) dst[k].v[i] = 0.f;
            }
        }
    };

    // Row ends of the next 32 rows, relative to e0, one per lane.
    auto load_row_ends = [&](int base) -> int {
        const int row = base + lane;
        if (row < r1) return (int)(rowptr[row + 1] - e0);
        return INT_MAX;
    };
    int rbase = r;
    int row_ends = load_row_ends(rbase);
    int next_end = __shfl_sync(kFullMask, row_ends, 0);
    // Where the current row's nonzeros start, relative to e0: negative when the row began in an
    // earlier chunk.
    int row_start = 0;
    if (r < M) {
        const int64_t d = rowptr[r] - e0;
        row_start = d < 0 ? -1 : (int)d;
    }
    // The reference adds a row's terms onto the old output in order (old + a1*x1 + a2*x2 ...):
    // start the chain from the old row.  Only the chunk that FINISHES a row (r < r1) reads and
    // writes its Y, so a hub row cut across chunks has one reader/writer and no race; the chunks
    // before it start from zero and park their sums.
    // Rows without nonzeros are neither read nor written when accumulating (a remote or scatter
    // matrix leaves most rows empty): row r+1 is known to be empty when its end equals row r's end.
    auto next_row_needs_y = [&]() -> bool {
        if (!ACC || r + 1 >= r1) return false;
        const int w = r + 1 - rbase;
        if (w >= 32) return true;  // its end is outside the prefetched window: fetch to be safe
        return __shfl_sync(kFullMask, row_ends, w) > next_end;
    };
    load_y((r < r1 && !(row_start >= 0 && next_end == row_start)) ? r : (int)M, acc);
    load_y(next_row_needs_y() ? r + 1 : (int)M, ynext);

    auto advance_row = [&]() {
        row_start = next_end;
        ++r;
        if (r - rbase == 32) {
            rbase = r;
            row_ends = load_row_ends(rbase);
        }
        next_end = __shfl_sync(kFullMask, row_ends, r - rbase);
#pragma unroll
        for (int k = 0; k < NV; ++k) acc[k] = ynext[k];
        load_y(next_row_needs_y() ? r + 1 : (int)M, ynext);
    };

    // Packing epilogue: consecutive rows share a packed row (8 / PK rows per byte), and a warp meets them one
    // after the other, so the codes of the packed row in progress are merged in registers.  A packed row
    // whose rows were all encoded here is written with one plain store; one that is shared with another
    // chunk, or with a row the fix-up kernel finishes, is OR-ed into the zero-filled buffer.
    int pend_R = -1, pend_n = 0, pend_cnt = 0;
    uint32_t pend_w[PK ? NV : 1];
    auto flush_pending = [&]() {
        if (PK && pend_R >= 0 && grp == 0) {
            uint32_t *out = reinterpret_cast<uint32_t *>(pk.codes + (int64_t)pend_R * pk.F);
#pragma unroll
            for (int k = 0; k < (PK ? NV : 1); ++k)
                if (vok[k]) {
                    if (pend_n == pend_cnt)
                        __stcs(out + gl + k * G, pend_w[k]);
                    else if (pend_w[k] != 0u)
                        atomicOr(out + gl + k * G, pend_w[k]);
                }
        }
        pend_R = -1;
    };

    // Fold the S lane groups and write row r (its last nonzero is in this chunk).
    auto flush_row = [&]() {
        if (S > 1) {
#pragma unroll
            for (int off = G; off < 32; off <<= 1)
#pragma unroll
                for (int k = 0; k < NV; ++k)
#pragma unroll
                    for (int i = 0; i < VW; ++i) acc[k].v[i] += __shfl_xor_sync(kFullMask, acc[k].v[i], off);
        }
        if (PK) {
            if (grp == 0) {
                if (row_start < 0) {  // the row began in an earlier chunk: the fix-up kernel finishes and encodes it
                    float *hp = pk.head + c * (int64_t)carry_ld;
#pragma unroll
                    for (int k = 0; k < NV; ++k)
                        if (vok[k]) vstore_plain<VW>(hp + voff[k], acc[k]);
                } else {
                    constexpr int PKB = PK ? PK : 8;
                    constexpr int PEPB = 8 / PKB;
                    const int pseg = find_segment(sseg, pk.P, r);
                    const int j = r - sseg[pseg];
                    float4 xv[1][NV];
#pragma unroll
                    for (int k = 0; k < NV; ++k)
                        xv[0][k] = make_float4(acc[k].v[0], acc[k].v[VW > 1 ? 1 : 0], acc[k].v[VW > 2 ? 2 : 0],
                                               acc[k].v[VW > 3 ? 3 : 0]);
                    const int R = pbase[pseg] + j / PEPB;
                    if (R != pend_R) {
                        flush_pending();
                        pend_R = R, pend_n = 0;
                        const int left = sseg[pseg + 1] - (sseg[pseg] + (j / PEPB) * PEPB);  // rows of this packed row
                        pend_cnt = left < PEPB ? left : PEPB;
#pragma unroll
                        for (int k = 0; k < (PK ? NV : 1); ++k) pend_w[k] = 0u;
                    }
                    uint32_t w[NV];
                    encode_row<PKB, NV, G>(xv, r, gl, FV, pk.F, pk.params, pk.params_bf16, (PEPB - 1 - j % PEPB) * PKB, w);
#pragma unroll
                    for (int k = 0; k < (PK ? NV : 1); ++k) pend_w[k] |= w[k];
                    if (++pend_n == pend_cnt) flush_pending();
                }
            }
            return;
        }
        // accumulating onto an empty row changes nothing: skip the store
        const bool untouched = acc_mode && row_start >= 0 && next_end == row_start;
        if (grp == 0 && !untouched) {
            float *yp = Y + (int64_t)r * ldy;
#pragma unroll
            for (int k = 0; k < NV; ++k)
                if (vok[k]) vstore_stream<VW>(yp + voff[k], acc[k]);
        }
    };

    // What one gather instruction brings in, per step u: the fp32 vectors, or the packed words plus
    // the slot's decode parameters.
    Vec<VW> xr[QB ? 1 : U][QB ? 1 : NV];
    uint32_t wq[QB ? U : 1][QB ? NV : 1];
    float av[U];
    uint32_t pq[QB ? U : 1];  // the slot's bf16 (zero_point, scale) pair, widened when applied
    int shq[QB ? U : 1];

    for (int tile = 0; tile < ntiles; ++tile) {
        const int eb = tile * kTile;
        if (tile + 1 < ntiles) {
            issue_tile(tile + 1);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncwarp();
        int *tcol = s_col[wib][tile & 1];
        const float *tval = s_val[wib][tile & 1];
        uint32_t *tprm = s_prm[QB ? wib : 0][tile & 1];
        const int in_batch = (n - eb) < kTile ? (n - eb) : kTile;
        if (QB) {
            // wire slot -> (packed row, bit position) and its bf16 parameters, once per nonzero
            for (int i = lane; i < in_batch; i += 32) {
                const int slot = tcol[i];
                const int pseg = find_segment(sseg, q.P, slot);
                const int j = slot - sseg[pseg];
                tprm[i] = __ldg(q.params + slot);
                tcol[i] = ((pbase[pseg] + j / EPB) << 3) | ((EPB - 1 - j % EPB) * QB);
            }
            __syncwarp();
        }
        const int nsteps = (in_batch + S - 1) / S;
        const int full_steps = in_batch / S;  // steps in which every lane group holds a nonzero

        auto fetch = [&](int u, int j, bool ok) {  // j: position of the nonzero inside the tile
            const int cc = tcol[j];
            av[u] = tval[j];
            if (QB) {
                pq[u] = tprm[j];
                shq[u] = cc & 7;
                const uint32_t *wp = reinterpret_cast<const uint32_t *>(q.codes + (int64_t)(cc >> 3) * q.F);
#pragma unroll
                for (int k = 0; k < NV; ++k)
                    if (ok && vok[k]) wq[u][k] = __ldg(wp + gl + k * G);
            } else {
                const float *xp = X + (int64_t)cc * ldx;
#pragma unroll
                for (int k = 0; k < NV; ++k)
                    if (ok && vok[k]) xr[u][k] = vload<VW>(xp + voff[k]);
            }
        };
        auto apply = [&](int u) {
#pragma unroll
            for (int k = 0; k < NV; ++k)
                if (vok[k]) {
                    if (QB) {
                        // four codes of one packed word: shift the row's bit field down, mask every
                        // byte, then splice each byte under the exponent of 2^23 -- the float
                        // 8388608 + code -- and subtract 2^23 (exact): no integer-to-float conversion
                        constexpr uint32_t kMask = ((1u << QB) - 1u) * 0x01010101u;
                        const uint32_t ws = (wq[u][k] >> shq[u]) & kMask;
                        const float zq_u = __uint_as_float(pq[u] << 16), sq_u = __uint_as_float(pq[u] & 0xffff0000u);
#pragma unroll
                        for (int i = 0; i < VW; ++i) {
                            const float m = __uint_as_float(__byte_perm(ws, 0x4B000000u, 0x7440 + i));
                            const float x = fmaf(m - 8388608.0f, sq_u, zq_u);
                            acc[k].v[i] = fmaf(av[u], x, acc[k].v[i]);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < VW; ++i) acc[k].v[i] = fmaf(av[u], xr[u][k].v[i], acc[k].v[i]);
                    }
                }
        };

        for (int s0 = 0; s0 < nsteps; s0 += U) {
            if (s0 + U <= full_steps && next_end >= eb + (s0 + U) * S) {
                // Fast path: the next U*S nonzeros all belong to the current row -- issue the U
                // gathers back to back, then the U FMA groups, with nothing else in between.
#pragma unroll
                for (int u = 0; u < U; ++u) fetch(u, (s0 + u) * S + grp, true);
#pragma unroll
                for (int u = 0; u < U; ++u) apply(u);
                continue;
            }
            // General path: a row ends inside these steps, or the batch runs out.
            bool ok[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = (s0 + u) * S + grp;  // position inside the tile
                ok[u] = j < in_batch;
                fetch(u, ok[u] ? j : 0, ok[u]);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                if (s0 + u < nsteps) {  // warp-uniform
                    const int step_end = eb + (s0 + u + 1) * S;
                    const int eg = eb + (s0 + u) * S + grp;
                    bool pending = ok[u];
                    while (next_end < step_end) {  // a row ends before this step's last nonzero
                        if (pending && eg < next_end) {
                            apply(u);
                            pending = false;
                        }
                        flush_row();
                        advance_row();
                    }
                    if (pending) apply(u);
                }
            }
        }
        __syncwarp();  // every lane is done with this tile before the copy of the tile after next lands in it
    }
    // Row ends that follow the chunk's last nonzero (including empty rows).
    while (r < r1) {
        flush_row();
        advance_row();
    }
    if (PK) flush_pending();
    // A hub row continues in the next chunk: park the partial sum.
    if (r1 < M && e1 > rowptr[r1]) {
        if (S > 1) {
#pragma unroll
            for (int off = G; off < 32; off <<= 1)
#pragma unroll
                for (int k = 0; k < NV; ++k)
#pragma unroll
                    for (int i = 0; i < VW; ++i) acc[k].v[i] += __shfl_xor_sync(kFullMask, acc[k].v[i], off);
        }
        if (grp == 0) {
            float *cp = carry + c * (int64_t)carry_ld;
#pragma unroll
            for (int k = 0; k < NV; ++k)
                if (vok[k]) vstore_plain<VW>(cp + voff[k], acc[k]);
        }
    }
}

// One warp per chunk; only the first chunk of a run of chunks that park partial sums for
// the same row does anything: it adds the run, in chunk order, onto the row.
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    spmm_fixup_kernel(const int64_t *__restrict__ rowptr, int64_t M, float *__restrict__ Y, int64_t ldy, int F,
                      const int64_t *__restrict__ chunk_nz, const int32_t *__restrict__ chunk_row, int64_t nchunks,
                      const float *__restrict__ carry, int carry_ld) {
    const int lane = threadIdx.x & 31;
    const int64_t c = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (c >= nchunks) return;
    const int row = chunk_row[c + 1];
    if (row >= M) return;
    const int64_t rs = rowptr[row];
    if (chunk_nz[c + 1] <= rs) return;                              // chunk c parks nothing
    if (c > 0 && chunk_row[c] == row && chunk_nz[c] > rs) return;  // chunk c-1 leads this run
    int64_t last = c;
    while (last + 1 < nchunks && chunk_row[last + 2] == row) ++last;  // chunks c..last all park into `row`
    float *yp = Y + (int64_t)row * ldy;
    for (int f = lane; f < F; f += 32) {
        float s = 0.f;
        for (int64_t j = c; j <= last; ++j) s += carry[j * (int64_t)carry_ld + f];
        yp[f] += s;
    }
}

// Packing twin of the fix-up kernel: the first chunk of a run that parks into `row` adds the run's parked
// sums in chunk order onto the tail the finishing chunk left in `head` (the same additions, in the same
// order, as spmm_fixup_kernel applies to Y) and encodes the row.
template <int BITS>
__global__ void __launch_bounds__(kWarpsPerBlock * 32)
    spmm_fixup_pack_kernel(const int64_t *__restrict__ rowptr, int64_t M, const int64_t *__restrict__ chunk_nz,
                           const int32_t *__restrict__ chunk_row, int64_t nchunks, const float *__restrict__ carry,
                           int carry_ld, PackOut pk) {
    constexpr int EPB = 8 / BITS;
    __shared__ int sseg[kMaxSeg + 1];
    __shared__ int pbase[kMaxSeg + 1];
    build_packed_prefix(pk.seg, pk.P, EPB, pbase, sseg);
    const int lane = threadIdx.x & 31;
    const int64_t c = (int64_t)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    if (c >= nchunks) return;
    const int row = chunk_row[c + 1];
    if (row >= M) return;
    const int64_t rs = rowptr[row];
    if (chunk_nz[c + 1] <= rs) return;                              // chunk c parks nothing
    if (c > 0 && chunk_row[c] == row && chunk_nz[c] > rs) return;  // chunk c-1 leads this run
    int64_t last = c;
    while (last + 1 < nchunks && chunk_row[last + 2] == row) ++last;  // chunks c..last all park into `row`
    const int FV = pk.F >> 2;
    float4 xv[1][4];
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        const int vi = lane + 32 * k;
        xv[0][k] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (vi < FV) {
            float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int64_t j = c; j <= last; ++j) {
                const float4 t = *(reinterpret_cast<const float4 *>(carry + j * (int64_t)carry_ld) + vi);
                sum.x += t.x, sum.y += t.y, sum.z += t.z, sum.w += t.w;
            }
            const float4 h = *(reinterpret_cast<const float4 *>(pk.head + (last + 1) * (int64_t)carry_ld) + vi);
            xv[0][k] = make_float4(h.x + sum.x, h.y + sum.y, h.z + sum.z, h.w + sum.w);
        }
    }
    const int pseg = find_segment(sseg, pk.P, row);
    const int j = row - sseg[pseg];
    uint32_t w[4];
    const int64_t R = (int64_t)pbase[pseg] + j / EPB;
    quant_pack_group<BITS, 4, 32, 1>(xv, 1, row, R, lane, kFullMask, 0, FV, pk.F, 0, pk.params, pk.params_bf16, pk.codes,
                                     (EPB - 1 - j % EPB) * BITS, w);
    uint32_t *out = reinterpret_cast<uint32_t *>(pk.codes + R * pk.F);
#pragma unroll
    for (int k = 0; k < 4; ++k)
        if (lane + 32 * k < FV && w[k] != 0u) atomicOr(out + lane + 32 * k, w[k]);
}

// Zero fill of exactly the packed rows the segments need (their number lives on the device).
__global__ void zero_codes_kernel(const int32_t *__restrict__ seg, int P, int epb, int F, uint8_t *__restrict__ codes) {
    __shared__ int pbase[kMaxSeg + 1];
    build_packed_prefix(seg, P, epb, pbase);
    const int64_t words = (int64_t)pbase[P] * (F >> 2);
    uint32_t *w = reinterpret_cast<uint32_t *>(codes);
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < words; i += (int64_t)gridDim.x * blockDim.x) w[i] = 0u;
}

__global__ void csr_validate_kernel(const int64_t *__restrict__ rowptr, const int32_t *__restrict__ col, int64_t M,
                                    int64_t K, int64_t nnz, int32_t *status) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    int bad = 0;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i <= M; i += stride) {
        const int64_t v = rowptr[i];
        if (i == 0 && v != 0) bad |= 1;
        if (i == M && v != nnz) bad |= 1;
        if (i < M && (v > rowptr[i + 1] || v < 0)) bad |= 1;
    }
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += stride) {
        const int32_t cidx = col[e];
        if (cidx < 0 || cidx >= K) bad |= 2;
    }
    if (bad) atomicOr(status, bad);
}

template <int G, int NV, int VW, int U>
static void launch_chunks(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, const float *X,
                          int64_t ldx, float *Y, int64_t ldy, int FV, int accumulate, const int64_t *chunk_nz,
                          const int32_t *chunk_row, int64_t nchunks, float *carry, int carry_ld, int qbits,
                          const PackedOperand &q, int pkbits, const PackOut &pk, cudaStream_t st) {
    const unsigned blocks = (unsigned)div_up(nchunks, kWarpsPerBlock);
    const bool full = (FV == G * NV) && VW == 4;
    if (VW == 4 && pkbits != 0) {  // packing epilogue: fp32 operand, no accumulation, 128-bit path only
#define GNNAGG_GO_PK(FULL, PK)                                                                                  \
    spmm_chunk_kernel<G, NV, VW, U, false, FULL, 0, (VW == 4 ? PK : 0)><<<blocks, kWarpsPerBlock * 32, 0, st>>>( \
        rowptr, col, val, M, X, ldx, Y, ldy, FV, chunk_nz, chunk_row, nchunks, carry, carry_ld, q, pk)
        if (pkbits == 2) {
            if (full) GNNAGG_GO_PK((VW == 4), 2); else GNNAGG_GO_PK(false, 2);
        } else if (pkbits == 4) {
            if (full) GNNAGG_GO_PK((VW == 4), 4); else GNNAGG_GO_PK(false, 4);
        } else {
            if (full) GNNAGG_GO_PK((VW == 4), 8); else GNNAGG_GO_PK(false, 8);
        }
#undef GNNAGG_GO_PK
        return;
    }
    // a packed gather is 4 bytes per lane instead of 16: where registers allow, keep more in flight
    constexpr int UQ = NV == 2 ? 8 : U;  // F in (128, 256]: eight packed gathers in flight instead of four
#define GNNAGG_GO(ACC, FULL, QB)                                                                              \
    spmm_chunk_kernel<G, NV, VW, (QB ? UQ : U), ACC, FULL, QB, 0><<<blocks, kWarpsPerBlock * 32, 0, st>>>(    \
        rowptr, col, val, M, X, ldx, Y, ldy, FV, chunk_nz, chunk_row, nchunks, carry, carry_ld, q, pk)
    if (VW == 4 && qbits != 0) {  // packed operand: 128-bit path only, per-vector predicates kept
        if (qbits == 2) {
            if (accumulate) GNNAGG_GO(true, false, (VW == 4 ? 2 : 0)); else GNNAGG_GO(false, false, (VW == 4 ? 2 : 0));
        } else if (qbits == 4) {
            if (accumulate) GNNAGG_GO(true, false, (VW == 4 ? 4 : 0)); else GNNAGG_GO(false, false, (VW == 4 ? 4 : 0));
        } else {
            if (accumulate) GNNAGG_GO(true, false, (VW == 4 ? 8 : 0)); else GNNAGG_GO(false, false, (VW == 4 ? 8 : 0));
        }
    } else if (VW == 4 && full) {
        if (accumulate) GNNAGG_GO(true, (VW == 4), 0); else GNNAGG_GO(false, (VW == 4), 0);
    } else {
        if (accumulate) GNNAGG_GO(true, false, 0); else GNNAGG_GO(false, false, 0);
    }
#undef GNNAGG_GO
}

template <int VW>
static void dispatch_width(int FV, const int64_t *rowptr, const int32_t *col, const float *val, int64_t M,
                           const float *X, int64_t ldx, float *Y, int64_t ldy, int accumulate,
                           const int64_t *chunk_nz, const int32_t *chunk_row, int64_t nchunks, float *carry,
                           int carry_ld, int qbits, const PackedOperand &q, int pkbits, const PackOut &pk,
                           cudaStream_t st) {
#define GNNAGG_LAUNCH(G, NV, U)                                                                                 \
    launch_chunks<G, NV, VW, U>(rowptr, col, val, M, X, ldx, Y, ldy, FV, accumulate, chunk_nz, chunk_row, nchunks, \
                                carry, carry_ld, qbits, q, pkbits, pk, st)
    if (FV <= 2)
        GNNAGG_LAUNCH(2, 1, 2);
    else if (FV <= 4)
        GNNAGG_LAUNCH(4, 1, 4);
    else if (FV <= 8)
        GNNAGG_LAUNCH(8, 1, 8);
    else if (FV <= 16)
        GNNAGG_LAUNCH(16, 1, 8);
    else if (FV <= 32)
        GNNAGG_LAUNCH(32, 1, 8);
    else if (FV <= 64)
        GNNAGG_LAUNCH(32, 2, 4);
    else if (FV <= 96)
        GNNAGG_LAUNCH(32, 3, 2);
    else
        GNNAGG_LAUNCH(32, 4, 2);
#undef GNNAGG_LAUNCH
}

}  // namespace gnnagg

using namespace gnnagg;

extern "C" size_t gnnagg_spmm_plan_bytes(int64_t M, int64_t nnz) {
    if (M < 0 || nnz < 0) return 0;
    const int64_t nc = num_chunks(M, nnz, chunk_items());
    size_t b = sizeof(PlanHeader) + (size_t)(nc + 1) * (sizeof(int64_t) + sizeof(int32_t));
    return (b + 255) & ~(size_t)255;
}

extern "C" int gnnagg_spmm_plan_build(const int64_t *rowptr, int64_t M, int64_t nnz, void *plan, size_t plan_bytes,
                                      void *stream) {
    if (rowptr == nullptr || plan == nullptr || M < 0 || nnz < 0)
        return fail(GNNAGG_ERR_ARG, "spmm_plan_build: null pointer or negative size");
    if (M > INT32_MAX - 64) return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_plan_build: M must fit int32");
    if (plan_bytes < gnnagg_spmm_plan_bytes(M, nnz) || (reinterpret_cast<uintptr_t>(plan) & 7u))
        return fail(GNNAGG_ERR_SCRATCH, "spmm_plan_build: plan buffer too small or not 8-byte aligned");
    const int items = chunk_items();
    const int64_t nc = num_chunks(M, nnz, items);
    char *base = static_cast<char *>(plan);
    int64_t *cnz = reinterpret_cast<int64_t *>(base + sizeof(PlanHeader));
    int32_t *crow = reinterpret_cast<int32_t *>(cnz + (nc + 1));
    const int threads = 256;
    const unsigned blocks = (unsigned)div_up(nc + 1, threads);
    spmm_plan_kernel<<<blocks, threads, 0, static_cast<cudaStream_t>(stream)>>>(
        rowptr, M, nnz, items, nc, reinterpret_cast<PlanHeader *>(base), cnz, crow);
    return check_launch("spmm_plan_kernel");
}

// Widest column strip one launch covers: 128 vectors per row.
static int strip_floats(int vw) { return vw == 4 ? 512 : 128; }

extern "C" size_t gnnagg_spmm_scratch_bytes(int64_t M, int64_t nnz, int32_t F) {
    if (M < 0 || nnz < 0 || F <= 0) return 0;
    const int64_t nc = num_chunks(M, nnz, chunk_items());
    int ld = (F + 3) & ~3;
    if (ld > 512) ld = 512;
    return (((size_t)nc * ld * sizeof(float)) + 255) & ~(size_t)255;
}

// Shared body of the fp32-operand and packed-operand entry points.
static int spmm_launch(const char *who, const int64_t *rowptr, const int32_t *col, const float *val, int64_t M,
                       int64_t K, int64_t nnz, const float *X, int64_t ldx, float *Y, int64_t ldy, int32_t F,
                       int32_t accumulate, const void *plan, void *scratch, size_t scratch_bytes, int qbits,
                       PackedOperand q, void *stream) {
    if (M < 0 || K < 0 || nnz < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "%s: negative size", who);
    if (M == 0 || F == 0) return GNNAGG_OK;
    if (rowptr == nullptr || Y == nullptr || plan == nullptr) return fail(GNNAGG_ERR_ARG, "%s: null pointer", who);
    if (nnz > 0 && (col == nullptr || val == nullptr || (qbits == 0 && X == nullptr)))
        return fail(GNNAGG_ERR_ARG, "%s: null pointer", who);
    if ((qbits == 0 && ldx < F) || ldy < F) return fail(GNNAGG_ERR_ARG, "%s: leading dimension smaller than F", who);
    if (M > INT32_MAX - 64 || K > INT32_MAX) return fail(GNNAGG_ERR_UNSUPPORTED, "%s: M, K must fit int32", who);
    if (scratch == nullptr || scratch_bytes < gnnagg_spmm_scratch_bytes(M, nnz, F) || !aligned16(scratch))
        return fail(GNNAGG_ERR_SCRATCH, "%s: scratch missing, too small or not 16-byte aligned", who);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int items = chunk_items();
    const int64_t nc = num_chunks(M, nnz, items);
    const int64_t *cnz = plan_chunk_nz(plan);
    const int32_t *crow = plan_chunk_row(plan, nc);
    float *carry = static_cast<float *>(scratch);

    const bool vec4 = (F % 4 == 0) && (qbits != 0 || (ldx % 4 == 0 && aligned16(X))) && (ldy % 4 == 0) && aligned16(Y);
    if (qbits != 0 && !vec4)
        return fail(GNNAGG_ERR_UNSUPPORTED, "%s: packed operand needs F %% 4 == 0 and a 16-byte aligned output", who);
    const int vw = vec4 ? 4 : 1;
    const int strip = strip_floats(vw);
    for (int f0 = 0; f0 < F; f0 += strip) {
        const int fs = (F - f0) < strip ? (F - f0) : strip;
        const int carry_ld = (fs + 3) & ~3;
        const float *Xs = X == nullptr ? nullptr : X + f0;
        float *Ys = Y + f0;
        PackedOperand qs = q;
        if (qbits != 0) qs.codes = q.codes + f0;  // one byte per column: the strip starts f0 bytes into each packed row
        const PackOut nopack = {nullptr, nullptr, nullptr, nullptr, 0, 0, nullptr};
        if (vec4)
            dispatch_width<4>(fs / 4, rowptr, col, val, M, Xs, ldx, Ys, ldy, accumulate, cnz, crow, nc, carry, carry_ld,
                              qbits, qs, 0, nopack, st);
        else
            dispatch_width<1>(fs, rowptr, col, val, M, Xs, ldx, Ys, ldy, accumulate, cnz, crow, nc, carry, carry_ld, 0, qs,
                              0, nopack, st);
        int rc = check_launch("spmm_chunk_kernel");
        if (rc != GNNAGG_OK) return rc;
        spmm_fixup_kernel<<<(unsigned)div_up(nc, kWarpsPerBlock), kWarpsPerBlock * 32, 0, st>>>(
            rowptr, M, Ys, ldy, fs, cnz, crow, nc, carry, carry_ld);
        rc = check_launch("spmm_fixup_kernel");
        if (rc != GNNAGG_OK) return rc;
    }
    return GNNAGG_OK;
}

extern "C" int gnnagg_spmm_csr_f32(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                                   int64_t nnz, const float *X, int64_t ldx, float *Y, int64_t ldy, int32_t F,
                                   int32_t accumulate, const void *plan, void *scratch, size_t scratch_bytes,
                                   void *stream) {
    PackedOperand none = {nullptr, nullptr, nullptr, 0, 0};
    return spmm_launch("spmm", rowptr, col, val, M, K, nnz, X, ldx, Y, ldy, F, accumulate, plan, scratch, scratch_bytes,
                       0, none, stream);
}

extern "C" int gnnagg_spmm_csr_q(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                                 int64_t nnz, const uint8_t *codes, const void *params_bf16, const int32_t *seg,
                                 int32_t P, int32_t bits, float *Y, int64_t ldy, int32_t F, int32_t accumulate,
                                 const void *plan, void *scratch, size_t scratch_bytes, void *stream) {
    if (bits != 2 && bits != 4 && bits != 8) return fail(GNNAGG_ERR_ARG, "spmm_q: bits must be 2, 4 or 8");
    if (seg == nullptr || P < 1) return fail(GNNAGG_ERR_ARG, "spmm_q: bad seg / P");
    if (P > kMaxSeg) return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_q: more than %d segments", kMaxSeg);
    if (nnz > 0 && (codes == nullptr || params_bf16 == nullptr)) return fail(GNNAGG_ERR_ARG, "spmm_q: null pointer");
    if ((reinterpret_cast<uintptr_t>(codes) & 3u) || (reinterpret_cast<uintptr_t>(params_bf16) & 3u))
        return fail(GNNAGG_ERR_ARG, "spmm_q: codes and params must be 4-byte aligned");
    if (K > (INT32_MAX >> 3)) return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_q: too many wire slots");
    PackedOperand q = {codes, static_cast<const uint32_t *>(params_bf16), seg, P, F};
    return spmm_launch("spmm_q", rowptr, col, val, M, K, nnz, nullptr, 0, Y, ldy, F, accumulate, plan, scratch,
                       scratch_bytes, bits, q, stream);
}

extern "C" size_t gnnagg_spmm_quant_pack_scratch_bytes(int64_t M, int64_t nnz, int32_t F) {
    return 2 * gnnagg_spmm_scratch_bytes(M, nnz, F);  // parked sums of cut rows + the tails of the chunks that finish them
}

extern "C" int gnnagg_spmm_quant_pack(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                                      int64_t nnz, const float *X, int64_t ldx, int32_t F, const int32_t *seg,
                                      int32_t P, int32_t bits, float *params, void *params_bf16, uint8_t *codes,
                                      const void *plan, void *scratch, size_t scratch_bytes, void *stream) {
    if (M < 0 || K < 0 || nnz < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: negative size");
    if (bits != 2 && bits != 4 && bits != 8) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: bits must be 2, 4 or 8");
    if (seg == nullptr || P < 1) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: bad seg / P");
    if (P > kMaxSeg) return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_quant_pack: more than %d segments", kMaxSeg);
    if (M == 0 || F == 0) return GNNAGG_OK;
    if (rowptr == nullptr || params == nullptr || codes == nullptr || plan == nullptr ||
        (nnz > 0 && (col == nullptr || val == nullptr || X == nullptr)))
        return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: null pointer");
    if (ldx < F) return fail(GNNAGG_ERR_ARG, "spmm_quant_pack: ldx < F");
    if (M > INT32_MAX - 64 || K > INT32_MAX) return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_quant_pack: M, K must fit int32");
    const bool ok = (F % 4 == 0) && F <= 512 && (ldx % 4 == 0) && aligned16(X) &&
                    (reinterpret_cast<uintptr_t>(codes) % 4 == 0) && (reinterpret_cast<uintptr_t>(params) % 8 == 0) &&
                    (params_bf16 == nullptr || reinterpret_cast<uintptr_t>(params_bf16) % 4 == 0);
    if (!ok)
        return fail(GNNAGG_ERR_UNSUPPORTED,
                    "spmm_quant_pack: needs F %% 4 == 0, F <= 512 and 16-byte aligned dense rows; use gnnagg_spmm_csr_f32 "
                    "followed by gnnagg_quant_pack_rows");
    const size_t half = gnnagg_spmm_scratch_bytes(M, nnz, F);
    if (scratch == nullptr || scratch_bytes < 2 * half || !aligned16(scratch))
        return fail(GNNAGG_ERR_SCRATCH, "spmm_quant_pack: scratch missing, smaller than %zu bytes or not 16-byte aligned", 2 * half);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t nc = num_chunks(M, nnz, chunk_items());
    const int64_t *cnz = plan_chunk_nz(plan);
    const int32_t *crow = plan_chunk_row(plan, nc);
    float *carry = static_cast<float *>(scratch);
    const int carry_ld = (F + 3) & ~3;
    PackOut pk = {codes, params, static_cast<uint32_t *>(params_bf16), seg, P, F,
                  reinterpret_cast<float *>(static_cast<char *>(scratch) + half)};
    {  // packed rows shared between chunks (and rows finished by the fix-up kernel) are OR-ed in: start from zero
        zero_codes_kernel<<<kNumSMs * 4, 256, 0, st>>>(seg, P, 8 / bits, F, codes);
        const int rc0 = check_launch("zero_codes_kernel");
        if (rc0 != GNNAGG_OK) return rc0;
    }
    const PackedOperand none = {nullptr, nullptr, nullptr, 0, 0};
    dispatch_width<4>(F / 4, rowptr, col, val, M, X, ldx, nullptr, 0, 0, cnz, crow, nc, carry, carry_ld, 0, none, bits, pk, st);
    int rc = check_launch("spmm_chunk_kernel (packing epilogue)");
    if (rc != GNNAGG_OK) return rc;
    const unsigned fb = (unsigned)div_up(nc, kWarpsPerBlock);
    if (bits == 2) spmm_fixup_pack_kernel<2><<<fb, kWarpsPerBlock * 32, 0, st>>>(rowptr, M, cnz, crow, nc, carry, carry_ld, pk);
    else if (bits == 4) spmm_fixup_pack_kernel<4><<<fb, kWarpsPerBlock * 32, 0, st>>>(rowptr, M, cnz, crow, nc, carry, carry_ld, pk);
    else spmm_fixup_pack_kernel<8><<<fb, kWarpsPerBlock * 32, 0, st>>>(rowptr, M, cnz, crow, nc, carry, carry_ld, pk);
    return check_launch("spmm_fixup_pack_kernel");
}

extern "C" int gnnagg_csr_validate(const int64_t *rowptr, const int32_t *col, int64_t M, int64_t K, int64_t nnz,
                                   int32_t *status, void *stream) {
    if (rowptr == nullptr || status == nullptr || M < 0 || K < 0 || nnz < 0 || (nnz > 0 && col == nullptr))
        return fail(GNNAGG_ERR_ARG, "csr_validate: null pointer or negative size");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaMemsetAsync(status, 0, sizeof(int32_t), st);
    csr_validate_kernel<<<kNumSMs * 8, 256, 0, st>>>(rowptr, col, M, K, nnz, status);
    return check_launch("csr_validate_kernel");
}

// ---- SpMM variant for callers that cannot allocate device memory ----------------------------
// The partial-sum scratch of gnnagg_spmm_csr_f32 normally comes from the caller.  Some callers
// have no way to get device memory at the point of the call: code running under a framework
// whose allocator is off limits there, a plugin handed only its operands by the host
// application, or a process whose device-memory budget is fixed before it starts.  For them the
// scratch lives in a fixed buffer inside the library image; every GPU that loads the library
// holds GNNAGG_STATIC_SCRATCH_BYTES of it until the process exits.
namespace gnnagg {

static __device__ __align__(256) unsigned char g_static_scratch[GNNAGG_STATIC_SCRATCH_BYTES];

constexpr int kMaxDevices = 64;
static void *g_static_scratch_addr[kMaxDevices] = {nullptr};

// In host code `g_static_scratch` is only a handle for the symbol, not a device address: the
// address valid on the current device has to be asked for, once per device.
static int static_scratch_for_current_device(void **out) {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return fail(GNNAGG_ERR_CUDA, "spmm_static_scratch: cudaGetDevice: %s", cudaGetErrorString(e));
    if (dev < 0 || dev >= kMaxDevices)
        return fail(GNNAGG_ERR_UNSUPPORTED, "spmm_static_scratch: device ordinal %d out of range", dev);
    void *p = __atomic_load_n(&g_static_scratch_addr[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || p == nullptr)
            return fail(GNNAGG_ERR_CUDA, "spmm_static_scratch: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
        __atomic_store_n(&g_static_scratch_addr[dev], p, __ATOMIC_RELEASE);  // same value from any thread
    }
    *out = p;
    return GNNAGG_OK;
}

}  // namespace gnnagg

extern "C" int gnnagg_spmm_csr_f32_static_scratch(const int64_t *rowptr, const int32_t *col, const float *val,
                                                  int64_t M, int64_t K, int64_t nnz, const float *X, int64_t ldx,
                                                  float *Y, int64_t ldy, int32_t F, int32_t accumulate,
                                                  const void *plan, void *stream) {
    if (M < 0 || K < 0 || nnz < 0 || F < 0) return fail(GNNAGG_ERR_ARG, "spmm_static_scratch: negative size");
    if (M == 0 || F == 0) return GNNAGG_OK;
    const size_t need = gnnagg_spmm_scratch_bytes(M, nnz, F);
    if (need > (size_t)GNNAGG_STATIC_SCRATCH_BYTES)
        return fail(GNNAGG_ERR_SCRATCH,
                    "spmm_static_scratch: this product needs %zu bytes of scratch but the built-in buffer holds %zu; "
                    "use gnnagg_spmm_csr_f32 with caller-provided scratch",
                    need, (size_t)GNNAGG_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != GNNAGG_OK) return rc;
    return gnnagg_spmm_csr_f32(rowptr, col, val, M, K, nnz, X, ldx, Y, ldy, F, accumulate, plan, scratch,
                               (size_t)GNNAGG_STATIC_SCRATCH_BYTES, stream);
}
