// Dense feature transform on the 5th-generation tensor cores (tcgen05 + TMEM + TMA), sm_100a only:
//
//     C[M,N] (+)= A[M,K] . B[N,K]^T (+ bias[N])          all fp32, row-major, B = an nn.Linear weight
//
// in fp32-grade accuracy: every operand is split into two TF32 pieces, x = hi + lo, and three
// tensor-core products a_hi.b_lo + a_hi.b_hi + a_lo.b_hi are accumulated in fp32 in tensor memory (the
// dropped a_lo.b_lo term is below 2^-21 relative).  The weight is split once per call by a small
// kernel into a caller-provided workspace (hi = tf32_rna(w), lo = tf32_rna(w - hi)).  The activation
// panel is used as loaded for its "hi" products (the tensor core reads the upper 19 bits of an fp32
// word, i.e. hi = x truncated); its remainder panel lo = tf32_rna(x - hi) is computed inside the GEMM,
// in shared memory, while those products already run.  The tensor-memory accumulator rounds toward
// zero once per MMA, so the main product and the two small ones are kept in separate accumulators
// (the small ones' rounding errors are 2^-11 of the main one's) and added in the epilogue: measured
// error 3.7e-7 of sum |a||b| at K = 256 (an fp32 FMA chain: 3e-7; one shared accumulator: 1.3e-6).
//
// One persistent CTA per SM, 10 warps:
//   warp 0      lane 0 issues the TMA loads (A as stored, B_hi, B_lo per 32-wide k-block; two stages) and
//               prefetches the next row panel of A into L2;
//   warp 1      allocates tensor memory; lane 0 issues tcgen05.mma (128 x 128 x 8 per instruction, one
//               accumulator pair per 128 output columns) and the commits that free a stage / publish
//               the accumulators of a row panel;
//   warps 2-5   compute the remainder (lo) panel of a stage's A tile into a second buffer;
//   warps 6-9   epilogue: tcgen05.ld of the finished accumulators, main + small, bias add, 32 x 32
//               blocks through swizzled shared memory to TMA stores (TMA reduce-add for accumulate);
//               output rows that TMA cannot address go through a shared-memory transpose and plain
//               stores.  For N <= 128 two row panels fit in tensor memory and the epilogue of one runs
//               under the MMAs of the next.
// Every wait is bounded (about a second); on a time-out the kernel records a code in the status
// word of the workspace, drains its own copies and MMAs, frees tensor memory and returns.
#include <cuda.h>

#include <mutex>

#include "common.cuh"

namespace gnnagg {
namespace {

constexpr int BM = 128;                 // rows of A per tile = UMMA M = TMEM lanes
constexpr int BN = 128;                 // output columns per accumulator pair (N <= 256: one or two column halves)
constexpr int BK = 32;                  // fp32 per k-block: 128 bytes = one 128-byte swizzle row
constexpr int kRowBytes = BK * 4;
constexpr int UMMA_K = 8;               // tf32 elements per tcgen05.mma
constexpr int kStages = 2;
constexpr int kMaxN = 256;
constexpr int kTmemCols = 512;          // (main, small) accumulator pairs of 128 columns each: two column halves of
                                        // one row panel, or two row panels in flight when N <= 128
constexpr int kAccStride = 256;         // column offset of the second pair
constexpr int kSmallOffset = 128;       // column offset of a buffer's small-terms accumulator
constexpr int A_TILE_BYTES = BM * kRowBytes;     // 16 KB
constexpr int B_TILE_BYTES = kMaxN * kRowBytes;  // 32 KB per piece (all N rows of the weight)
constexpr int B_HALF_BYTES = BN * kRowBytes;     // the rows of one column half
constexpr int STAGE_BYTES = 2 * A_TILE_BYTES + 2 * B_TILE_BYTES;  // a (loaded), a_lo, b_hi, b_lo: 96 KB
constexpr int kEpiPad = 33;
constexpr int kEpiTile = 32 * 32 * 4;   // one 32 x 32 fp32 output block
constexpr int EPI_BYTES = 4 * 2 * kEpiTile;  // per epilogue warp: two blocks (TMA store double buffer)
constexpr int BIAS_BYTES = kMaxN * 4;
constexpr int kNumBarriers = 3 * kStages + 4 + 1;
constexpr int SMEM_BYTES = 1024 + kStages * STAGE_BYTES + EPI_BYTES + BIAS_BYTES + 256;
constexpr int kThreads = 320;
constexpr unsigned long long kWaitLimitNs = 1000ull * 1000ull * 1000ull;  // every launch but the stall test's
constexpr int kStatusBytes = 256;

static_assert(SMEM_BYTES <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ unsigned long long globaltimer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false when another role has raised `abort_flag` or when this wait ran out
// of time (it then raises the flag and leaves `code` in the status word, first writer wins).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status,
                                          int code, unsigned long long limit_ns) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = globaltimer_ns();
    uint32_t n = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++n & 31u) == 0) {
            if (*abort_flag != 0) return false;
            if (globaltimer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                atomicCAS(status, 0, code);
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cta.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
        "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_2d(const CUtensorMap *map, int x, int y) {
    asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(map), "r"(x), "r"(y) : "memory");
}

// Shared -> global tile store / add through the tensor map (rows and columns outside the tensor are clipped).
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(src),
                 "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_reduce_add_2d(const CUtensorMap *map, uint32_t src, int x, int y) {
    asm volatile("cp.reduce.async.bulk.tensor.2d.global.shared::cta.add.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map),
                 "r"(src), "r"(x), "r"(y)
                 : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int kPending>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(kPending) : "memory");
}
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_generic_to_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                            uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(tmem_d),
        "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// 32 lanes x 32 columns of fp32: thread t of the warp receives columns [c, c+32) of TMEM lane
// (lane base of the address) + t.
__device__ __forceinline__ void tc_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
          "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
          "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
          "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ float tf32_rna(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
}

__device__ __forceinline__ void split_tf32(float x, float &hi, float &lo) {
    hi = tf32_rna(x);
    const float rest = x - hi;  // exact
    lo = (fabsf(hi) <= 3.402823466e38f) ? tf32_rna(rest) : 0.0f;  // inf / nan stay in hi alone
}

// The activation panel is used as loaded for the "hi" products: the tensor core reads the upper 19
// bits of each fp32 word, i.e. hi = x with the low 13 mantissa bits cut.  lo is the remainder.
__device__ __forceinline__ float lo_of_truncated(float x) {
    const float hi = __uint_as_float(__float_as_uint(x) & 0xFFFFE000u);
    const float rest = x - hi;  // exact
    return (fabsf(hi) <= 3.402823466e38f) ? tf32_rna(rest) : 0.0f;
}

// Shared-memory matrix descriptor of a K-major tile whose rows are 128 bytes, 128-byte-swizzled (what
// TMA writes for a {32 fp32, rows} box): start address, 8-row group stride 1024 bytes, descriptor
// version 1 (sm_100), layout type 2 (128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // bits [0,14)
    d |= (uint64_t)1 << 16;                              // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;                    // stride byte offset
    d |= (uint64_t)1 << 46;                              // descriptor version
    d |= (uint64_t)2 << 61;                              // SWIZZLE_128B
    return d;
}

// Instruction descriptor of kind::tf32: fp32 accumulator, TF32 A and B, both K-major, M = 128.
__host__ __device__ inline uint32_t make_instr_desc(int n) {
    uint32_t d = 0;
    d |= 1u << 4;                    // D format: f32
    d |= 2u << 7;                    // A format: tf32
    d |= 2u << 10;                   // B format: tf32
    d |= (uint32_t)(n >> 3) << 17;   // N / 8
    d |= (uint32_t)(BM >> 4) << 24;  // M / 16
    return d;
}

struct GemmParams {
    float *C;
    const float *bias;
    int *status;
    int64_t M, ldc;
    int N, n_pad, K, accumulate, num_tiles, tma_store, b_box_rows;
    unsigned long long wait_ns;  // limit of every wait
    uint32_t tx_excess;          // bytes announced to the load barrier beyond what the loads deliver (stall test only)
};

enum : int {
    kErrWaitEmpty = 1,      // TMA issuer waited for a free stage
    kErrWaitFull = 2,       // split warps waited for a TMA load
    kErrWaitSplit = 3,      // MMA issuer waited for the split tile
    kErrWaitAccFree = 4,    // MMA issuer waited for the epilogue to release an accumulator
    kErrWaitAccFull = 5,    // epilogue waited for an accumulator
    kErrDrain = 6,          // bounded drain after an abort ran out
};

__global__ void __launch_bounds__(kThreads, 1)
gemm_tf32x3_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_bhi,
                   const __grid_constant__ CUtensorMap map_blo, const __grid_constant__ CUtensorMap map_c,
                   const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment: the swizzle pattern and the descriptors assume it
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint8_t *stage_base = smem;
    uint8_t *epi = smem + kStages * STAGE_BYTES;
    float *bias_s = reinterpret_cast<float *>(smem + kStages * STAGE_BYTES + EPI_BYTES);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + kStages * STAGE_BYTES + EPI_BYTES + BIAS_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + kNumBarriers);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto bar_split = [&](int s) { return bar0 + 8u * (uint32_t)(kStages + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * kStages + s); };
    auto bar_acc_full = [&](int b) { return bar0 + 8u * (uint32_t)(3 * kStages + b); };
    auto bar_acc_empty = [&](int b) { return bar0 + 8u * (uint32_t)(3 * kStages + 2 + b); };
    const uint32_t bar_drain = bar0 + 8u * (uint32_t)(3 * kStages + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KB = (p.K + BK - 1) / BK;
    const int halves = (p.n_pad + BN - 1) / BN;  // column halves of a row panel: 1 or 2
    const int nbuf = halves == 1 ? 2 : 1;         // row panels whose accumulators fit in tensor memory at once
    const uint32_t b_bytes = (uint32_t)p.b_box_rows * kRowBytes;
    for (int i = threadIdx.x; i < kMaxN; i += kThreads) bias_s[i] = (p.bias != nullptr && i < p.N) ? p.bias[i] : 0.0f;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_split(s), 128);
            mbar_init(bar_empty(s), 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(bar_acc_full(b), 1);
            mbar_init(bar_acc_empty(b), 128);
        }
        mbar_init(bar_drain, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
                const int m0 = tile * BM;
                const int next = tile + (int)gridDim.x;
                if (next < p.num_tiles)
                    for (int kb = 0; kb < KB; ++kb) tma_prefetch_2d(&map_a, kb * BK, next * BM);
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, p.status, kErrWaitEmpty, p.wait_ns)) {
                        ok = false;
                        break;
                    }
                    const uint32_t sa = smem_u32(stage_base + s * STAGE_BYTES);
                    mbar_arrive_expect_tx(bar_full(s), (uint32_t)A_TILE_BYTES + 2u * b_bytes + p.tx_excess);
                    tma_load_2d(sa, &map_a, bar_full(s), kb * BK, m0);
                    tma_load_2d(sa + 2 * A_TILE_BYTES, &map_bhi, bar_full(s), kb * BK, 0);
                    tma_load_2d(sa + 2 * A_TILE_BYTES + B_TILE_BYTES, &map_blo, bar_full(s), kb * BK, 0);
                }
            }
            if (!ok) {
                // copies of the last k-blocks issued may still be landing: wait for them, bounded
                for (uint32_t back = 1; back <= (uint32_t)kStages && back <= it; ++back) {
                    const uint32_t j = it - back;
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar_full(j % kStages), (j / kStages) & 1u)) {
                        if (globaltimer_ns() - t0 > p.wait_ns) {
                            atomicCAS(p.status, 0, (int)kErrDrain);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            uint32_t it = 0, t = 0;
            bool ok = true;
            uint32_t idesc[2];
            for (int h = 0; h < 2; ++h) idesc[h] = make_instr_desc(max(16, min(BN, p.n_pad - h * BN)));
            for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++t) {
                const int b = (int)(t % (uint32_t)nbuf);
                if (!mbar_wait(bar_acc_empty(b), ((t / (uint32_t)nbuf) & 1u) ^ 1u, abort_flag, p.status,
                               kErrWaitAccFree, p.wait_ns)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                // the main product and the two small ones have accumulators of their own: the accumulator
                // rounds toward zero once per MMA, and the small terms would otherwise triple the number of
                // roundings at full magnitude.  Column half h of row-panel buffer b sits at pair (b + h).
                for (int kb = 0; kb < KB; ++kb, ++it) {
                    const int s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1u;
                    if (!mbar_wait(bar_full(s), ph, abort_flag, p.status, kErrWaitFull, p.wait_ns)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t sa = smem_u32(stage_base + s * STAGE_BYTES);
                    const uint64_t a_hi = make_smem_desc(sa);  // the panel as loaded
                    const uint64_t a_lo = make_smem_desc(sa + A_TILE_BYTES);
                    const uint32_t first = (kb > 0) ? 1u : 0u;
                    // the two products of the loaded panel start at once; k advances 32 bytes inside the swizzled row
                    for (int h = 0; h < halves; ++h) {
                        const uint32_t d_main = tmem_base + (uint32_t)((b + h) * kAccStride);
                        const uint32_t d_small = d_main + (uint32_t)kSmallOffset;
                        const uint64_t b_hi = make_smem_desc(sa + 2 * A_TILE_BYTES + h * B_HALF_BYTES);
                        const uint64_t b_lo = make_smem_desc(sa + 2 * A_TILE_BYTES + B_TILE_BYTES + h * B_HALF_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tc_mma_tf32(d_small, a_hi + (uint64_t)(2 * k), b_lo + (uint64_t)(2 * k), idesc[h],
                                        k > 0 ? 1u : first);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tc_mma_tf32(d_main, a_hi + (uint64_t)(2 * k), b_hi + (uint64_t)(2 * k), idesc[h],
                                        k > 0 ? 1u : first);
                    }
                    // the remainder panel is ready a little later
                    if (!mbar_wait(bar_split(s), ph, abort_flag, p.status, kErrWaitSplit, p.wait_ns)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    for (int h = 0; h < halves; ++h) {
                        const uint32_t d_small = tmem_base + (uint32_t)((b + h) * kAccStride + kSmallOffset);
                        const uint64_t b_hi = make_smem_desc(sa + 2 * A_TILE_BYTES + h * B_HALF_BYTES);
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k)
                            tc_mma_tf32(d_small, a_lo + (uint64_t)(2 * k), b_hi + (uint64_t)(2 * k), idesc[h], 1u);
                    }
                    tc_commit(bar_empty(s));  // the stage is free once these MMAs have read it
                }
                if (ok) tc_commit(bar_acc_full(b));
            }
            if (!ok) {
                // MMAs already issued still read shared memory and write tensor memory: drain, bounded
                tc_commit(bar_drain);
                const unsigned long long t0 = globaltimer_ns();
                while (!mbar_try_wait(bar_drain, 0)) {
                    if (globaltimer_ns() - t0 > p.wait_ns) {
                        atomicCAS(p.status, 0, (int)kErrDrain);
                        break;
                    }
                }
            }
        }
    } else if (warp < 6) {
        // ---------------- split warps: remainder panel of the loaded A tile ----------------
        const int tid = threadIdx.x - 64;  // 0..127
        uint32_t it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x) {
            for (int kb = 0; kb < KB; ++kb, ++it) {
                const int s = it % kStages;
                const uint32_t ph = (it / kStages) & 1u;
                if (!mbar_wait(bar_full(s), ph, abort_flag, p.status, kErrWaitFull, p.wait_ns)) {
                    ok = false;
                    break;
                }
                const float4 *raw = reinterpret_cast<const float4 *>(stage_base + s * STAGE_BYTES);
                float4 *lo = reinterpret_cast<float4 *>(stage_base + s * STAGE_BYTES + A_TILE_BYTES);
#pragma unroll
                for (int j = 0; j < A_TILE_BYTES / 16 / 128; ++j) {
                    const int i = tid + 128 * j;
                    const float4 v = raw[i];
                    float4 l;
                    l.x = lo_of_truncated(v.x);
                    l.y = lo_of_truncated(v.y);
                    l.z = lo_of_truncated(v.z);
                    l.w = lo_of_truncated(v.w);
                    lo[i] = l;
                }
                fence_generic_to_async_smem();
                mbar_arrive(bar_split(s));
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        const int q = warp & 3;  // TMEM lane quarter this warp may read
        uint8_t *my_epi = epi + (warp - 6) * 2 * kEpiTile;  // 1024-byte aligned
        float *tr = reinterpret_cast<float *>(my_epi);
        uint32_t t = 0, nstore = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < p.num_tiles && ok; tile += gridDim.x, ++t) {
            const int64_t row0 = (int64_t)tile * BM + q * 32;
            const int b = (int)(t % (uint32_t)nbuf);
            // warp-uniform outcome: the tensor-memory loads below are warp-collective
            if (!__all_sync(kFullMask, mbar_wait(bar_acc_full(b), (t / (uint32_t)nbuf) & 1u, abort_flag, p.status,
                                                 kErrWaitAccFull, p.wait_ns))) {
                ok = false;
                break;
            }
            tc_fence_after();
            for (int h = 0; h < halves; ++h) {
                const int col_base = h * BN;
                const int n_valid = min(BN, p.N - col_base);
                const uint32_t t_main = tmem_base + (uint32_t)((b + h) * kAccStride) + ((uint32_t)(q * 32) << 16);
                for (int c0 = 0; c0 < n_valid; c0 += 32) {
                    uint32_t r[32], rs[32];
                    tc_ld_32x32(t_main + (uint32_t)c0, r);
                    tc_ld_32x32(t_main + (uint32_t)(kSmallOffset + c0), rs);
                    float v[32];
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]) + __uint_as_float(rs[j]);
                    if (p.tma_store) {
                        // this thread's row of the 32 x 32 block goes to shared memory in the 128-byte-swizzled
                        // layout of the output tensor map (16-byte chunk j of row r sits at chunk j ^ (r & 7)),
                        // then one lane hands the block to TMA: plain store, or add for accumulate
                        uint8_t *buf = my_epi + (nstore & 1u) * kEpiTile;
                        if (lane == 0) tma_store_wait_read<1>();  // the store that last read this buffer is done
                        __syncwarp();
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            float4 o;
                            o.x = v[4 * j + 0] + bias_s[col_base + c0 + 4 * j + 0];
                            o.y = v[4 * j + 1] + bias_s[col_base + c0 + 4 * j + 1];
                            o.z = v[4 * j + 2] + bias_s[col_base + c0 + 4 * j + 2];
                            o.w = v[4 * j + 3] + bias_s[col_base + c0 + 4 * j + 3];
                            *reinterpret_cast<float4 *>(buf + lane * 128 + ((j ^ (lane & 7)) << 4)) = o;
                        }
                        fence_generic_to_async_smem();
                        __syncwarp();
                        if (lane == 0) {
                            if (p.accumulate)
                                tma_reduce_add_2d(&map_c, smem_u32(buf), col_base + c0, (int)row0);
                            else
                                tma_store_2d(&map_c, smem_u32(buf), col_base + c0, (int)row0);
                            tma_store_commit();
                        }
                        ++nstore;
                        continue;
                    }
                    // output rows that TMA cannot address (stride not a multiple of 16 bytes): transpose the
                    // block through shared memory and store row segments with plain coalesced stores
#pragma unroll
                    for (int j = 0; j < 32; ++j) tr[lane * kEpiPad + j] = v[j];
                    __syncwarp();
                    const int col = col_base + c0 + lane;
                    if (col < p.N) {
                        const float bv = bias_s[col];
#pragma unroll 4
                        for (int rr = 0; rr < 32; ++rr) {
                            const int64_t row = row0 + rr;
                            if (row >= p.M) break;
                            float o = tr[rr * kEpiPad + lane] + bv;
                            float *dst = p.C + row * p.ldc + col;
                            if (p.accumulate) o += *dst;
                            *dst = o;
                        }
                    }
                    __syncwarp();
                }
            }
            tc_fence_before();
            mbar_arrive(bar_acc_empty(b));
        }
        if (p.tma_store && lane == 0) tma_store_wait_all();  // shared memory stays valid until TMA has read it
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

// ---------------------------------------------------------------------------------------------
// Weight gradient  dW[N,K] = G[M,N]^T . X[M,K]: a reduction over all M rows into a small matrix.
//
// Both operands are "MN-major" for the tensor core (the reduction index, the row, is the slow
// dimension in memory), which tcgen05 takes directly.  For 32-bit elements that needs the 128-byte
// swizzle with 32-byte atoms, both in the tensor map (SWIZZLE_128B_ATOM_32B) and in the shared-memory
// descriptor (layout type 1; with the plain 128-byte swizzle the MMA returns zeros): a {32 columns,
// 16 rows} TMA box lands as 16 k-rows of 128 bytes, groups of 4 k-rows 512 bytes apart (stride byte
// offset), the boxes of one operand 2 KB apart (leading byte offset); one MMA consumes 8 k-rows.
// Each CTA owns a contiguous block of rows and accumulates its 256 x 256 partial product in tensor
// memory (two 128-lane halves).  The tensor-memory accumulator rounds toward zero once per MMA, a
// one-sided error that grows with the length of the chain, so every 2048 rows the accumulator is
// moved out and added (round to nearest, CUDA cores) to the CTA's partial in scratch; a second kernel
// adds the per-CTA partials in a fixed order.  The remainder (lo) panels of both operands are computed in shared memory as in
// the forward kernel; products: G.X + G_lo.X + G.X_lo.
constexpr int WG_ROWS = 16;                           // rows (k) per stage: two MMAs of k = 8
constexpr int WG_BOX_BYTES = WG_ROWS * 128;           // one {32 columns, 16 rows} box
constexpr int WG_PANEL_BYTES = 8 * WG_BOX_BYTES;      // up to 256 columns of one operand: 16 KB
constexpr int WG_STAGE_BYTES = 4 * WG_PANEL_BYTES;    // g, g_lo, x, x_lo
constexpr int WG_STAGES = 3;
constexpr int WG_FLUSH = 128;                         // stages (2048 rows) per accumulation block, see below
constexpr int WG_THREADS = 320;
constexpr int WG_SMEM_BYTES = 1024 + WG_STAGES * WG_STAGE_BYTES + 256;
static_assert(WG_SMEM_BYTES <= 227 * 1024, "shared memory budget");

__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t smem_addr, uint64_t tmpl) {
    return tmpl | (uint64_t)((smem_addr & 0x3FFFFu) >> 4);
}
// everything but the start address: leading / stride byte offsets, version 1, layout type
inline uint64_t smem_desc_mn_template(int lbo_bytes, int sbo_bytes, int layout) {
    uint64_t d = 0;
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(sbo_bytes >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)layout << 61;
    return d;
}

struct WgradParams {
    float *partial;   // [grid][n_rows][kp]
    int *status;
    int64_t M;
    int N, K, n_pad, kp, blocks_per_cta, total_blocks;
    uint64_t desc;   // shared-memory descriptor without the start address
    unsigned long long wait_ns;
    uint32_t tx_excess;
};

__global__ void __launch_bounds__(WG_THREADS, 1)
wgrad_tf32x3_kernel(const __grid_constant__ CUtensorMap map_g, const __grid_constant__ CUtensorMap map_x,
                    const WgradParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + WG_STAGES * WG_STAGE_BYTES);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 3 * WG_STAGES + 3);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    const uint32_t bar0 = smem_u32(bars);
    auto bar_full = [&](int s) { return bar0 + 8u * (uint32_t)s; };
    auto bar_split = [&](int s) { return bar0 + 8u * (uint32_t)(WG_STAGES + s); };
    auto bar_empty = [&](int s) { return bar0 + 8u * (uint32_t)(2 * WG_STAGES + s); };
    const uint32_t bar_acc = bar0 + 8u * (uint32_t)(3 * WG_STAGES);        // an accumulation block is complete
    const uint32_t bar_drain = bar0 + 8u * (uint32_t)(3 * WG_STAGES + 1);
    const uint32_t bar_flushed = bar0 + 8u * (uint32_t)(3 * WG_STAGES + 2);  // ... and has been moved out

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nb_g = (p.N + 31) / 32, nb_x = (p.n_pad + 31) / 32;   // boxes per operand
    const int halves = p.N > 128 ? 2 : 1;
    const int kb0 = blockIdx.x * p.blocks_per_cta;
    const int kb1 = min(kb0 + p.blocks_per_cta, p.total_blocks);
    const int nkb = kb1 - kb0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < WG_STAGES; ++s) {
            mbar_init(bar_full(s), 1);
            mbar_init(bar_split(s), 256);
            mbar_init(bar_empty(s), 1);
        }
        mbar_init(bar_acc, 1);
        mbar_init(bar_drain, 1);
        mbar_init(bar_flushed, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            bool ok = true;
            int it = 0;
            for (; it < nkb; ++it) {
                const int s = it % WG_STAGES;
                const uint32_t ph = (uint32_t)(it / WG_STAGES) & 1u;
                if (!mbar_wait(bar_empty(s), ph ^ 1u, abort_flag, p.status, kErrWaitEmpty, p.wait_ns)) {
                    ok = false;
                    break;
                }
                const uint32_t sa = smem_u32(smem + s * WG_STAGE_BYTES);
                const int row = (kb0 + it) * WG_ROWS;
                mbar_arrive_expect_tx(bar_full(s), (uint32_t)(nb_g + nb_x) * WG_BOX_BYTES + p.tx_excess);
                for (int b = 0; b < nb_g; ++b) tma_load_2d(sa + b * WG_BOX_BYTES, &map_g, bar_full(s), 32 * b, row);
                for (int b = 0; b < nb_x; ++b)
                    tma_load_2d(sa + 2 * WG_PANEL_BYTES + b * WG_BOX_BYTES, &map_x, bar_full(s), 32 * b, row);
            }
            if (!ok) {
                for (int back = 1; back <= WG_STAGES && back <= it; ++back) {
                    const int j = it - back;
                    const unsigned long long t0 = globaltimer_ns();
                    while (!mbar_try_wait(bar_full(j % WG_STAGES), (uint32_t)(j / WG_STAGES) & 1u)) {
                        if (globaltimer_ns() - t0 > p.wait_ns) {
                            atomicCAS(p.status, 0, (int)kErrDrain);
                            break;
                        }
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            // kind::tf32, fp32 accumulate, A and B both MN-major (bits 15, 16), M = 128, N = n_pad
            const uint32_t idesc = make_instr_desc(p.n_pad) | (1u << 15) | (1u << 16);
            bool ok = true;
            for (int it = 0; it < nkb; ++it) {
                const int s = it % WG_STAGES;
                const uint32_t ph = (uint32_t)(it / WG_STAGES) & 1u;
                const bool first = (it % WG_FLUSH) == 0;  // first stage of an accumulation block
                if (first && it > 0) {
                    // publish the finished block and wait until warps 2-5 have moved it out
                    tc_commit(bar_acc);
                    if (!mbar_wait(bar_flushed, (uint32_t)(it / WG_FLUSH - 1) & 1u, abort_flag, p.status,
                                   kErrWaitAccFree, p.wait_ns)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                }
                if (!mbar_wait(bar_full(s), ph, abort_flag, p.status, kErrWaitFull, p.wait_ns)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t sa = smem_u32(smem + s * WG_STAGE_BYTES);
                const uint32_t g_raw = sa, g_lo = sa + WG_PANEL_BYTES, x_raw = sa + 2 * WG_PANEL_BYTES,
                               x_lo = sa + 3 * WG_PANEL_BYTES;
#pragma unroll
                for (int ks = 0; ks < WG_ROWS / UMMA_K; ++ks)
                    for (int h = 0; h < halves; ++h)
                        tc_mma_tf32(tmem_base + (uint32_t)(h * kAccStride),
                                    make_smem_desc_mn(g_raw + h * 4 * WG_BOX_BYTES + ks * 1024, p.desc),
                                    make_smem_desc_mn(x_raw + ks * 1024, p.desc), idesc, (!first || ks > 0) ? 1u : 0u);
                if (!mbar_wait(bar_split(s), ph, abort_flag, p.status, kErrWaitSplit, p.wait_ns)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (int ks = 0; ks < WG_ROWS / UMMA_K; ++ks)
                    for (int h = 0; h < halves; ++h) {
                        const uint32_t d = tmem_base + (uint32_t)(h * kAccStride);
                        tc_mma_tf32(d, make_smem_desc_mn(g_lo + h * 4 * WG_BOX_BYTES + ks * 1024, p.desc),
                                    make_smem_desc_mn(x_raw + ks * 1024, p.desc), idesc, 1u);
                        tc_mma_tf32(d, make_smem_desc_mn(g_raw + h * 4 * WG_BOX_BYTES + ks * 1024, p.desc),
                                    make_smem_desc_mn(x_lo + ks * 1024, p.desc), idesc, 1u);
                    }
                tc_commit(bar_empty(s));
            }
            if (ok) {
                tc_commit(bar_acc);
            } else {
                tc_commit(bar_drain);
                const unsigned long long t0 = globaltimer_ns();
                while (!mbar_try_wait(bar_drain, 0)) {
                    if (globaltimer_ns() - t0 > p.wait_ns) {
                        atomicCAS(p.status, 0, (int)kErrDrain);
                        break;
                    }
                }
            }
        }
    } else {
        // ---- warps 2-9: remainder panels; warps 2-5 also move finished accumulation blocks out ----
        const int tid = threadIdx.x - 64;  // 0..255
        const int q = warp & 3;            // TMEM lane quarter of warps 2-5
        float *out = p.partial + (int64_t)blockIdx.x * p.N * p.kp;
        // block `fidx` of this CTA is complete in tensor memory: add it to the partial in scratch
        auto flush = [&](int fidx) -> bool {
            const bool ready = mbar_wait(bar_acc, (uint32_t)fidx & 1u, abort_flag, p.status, kErrWaitAccFull, p.wait_ns);
            if (!__all_sync(kFullMask, ready)) return false;
            tc_fence_after();
            for (int h = 0; h < halves; ++h) {
                const int n = h * 128 + q * 32 + lane;
                for (int c0 = 0; c0 < p.K; c0 += 32) {
                    uint32_t r[32];
                    tc_ld_32x32(tmem_base + (uint32_t)(h * kAccStride + c0) + ((uint32_t)(q * 32) << 16), r);
                    if (n < p.N) {
#pragma unroll
                        for (int j = 0; j < 8; ++j)
                            if (c0 + 4 * j < p.kp) {
                                float4 *dst = reinterpret_cast<float4 *>(out + (int64_t)n * p.kp + c0 + 4 * j);
                                float4 v = make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                       __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3]));
                                if (fidx > 0) {
                                    const float4 o = *dst;
                                    v.x += o.x, v.y += o.y, v.z += o.z, v.w += o.w;
                                }
                                *dst = v;
                            }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_flushed);
            return true;
        };
        bool ok = true;
        for (int it = 0; it < nkb; ++it) {
            if (warp < 6 && it > 0 && (it % WG_FLUSH) == 0 && !flush(it / WG_FLUSH - 1)) {
                ok = false;
                break;
            }
            const int s = it % WG_STAGES;
            const uint32_t ph = (uint32_t)(it / WG_STAGES) & 1u;
            if (!mbar_wait(bar_full(s), ph, abort_flag, p.status, kErrWaitFull, p.wait_ns)) {
                ok = false;
                break;
            }
            uint8_t *st = smem + s * WG_STAGE_BYTES;
            const int ng4 = nb_g * (WG_BOX_BYTES / 16), nx4 = nb_x * (WG_BOX_BYTES / 16);
            {
                const float4 *graw = reinterpret_cast<const float4 *>(st);
                float4 *glo = reinterpret_cast<float4 *>(st + WG_PANEL_BYTES);
                for (int i = tid; i < ng4; i += 256) {
                    const float4 v = graw[i];
                    glo[i] = make_float4(lo_of_truncated(v.x), lo_of_truncated(v.y), lo_of_truncated(v.z),
                                         lo_of_truncated(v.w));
                }
                const float4 *xraw = reinterpret_cast<const float4 *>(st + 2 * WG_PANEL_BYTES);
                float4 *xlo = reinterpret_cast<float4 *>(st + 3 * WG_PANEL_BYTES);
                for (int i = tid; i < nx4; i += 256) {
                    const float4 v = xraw[i];
                    xlo[i] = make_float4(lo_of_truncated(v.x), lo_of_truncated(v.y), lo_of_truncated(v.z),
                                         lo_of_truncated(v.w));
                }
            }
            fence_generic_to_async_smem();
            mbar_arrive(bar_split(s));
        }
        if (warp < 6 && ok) flush((nkb - 1) / WG_FLUSH);  // the last block
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)kTmemCols)
                     : "memory");
    }
}

// dW[n,k] = sum over CTAs of partial[cta][n][k], fixed order.
__global__ void wgrad_reduce_kernel(const float *__restrict__ partial, int nparts, int N, int K, int kp,
                                    float *__restrict__ dW, int64_t ldw) {
    const int total = N * K;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int n = i / K, k = i % K;
        const float *src = partial + (int64_t)n * kp + k;
        const int64_t step = (int64_t)N * kp;
        float s0 = 0.0f, s1 = 0.0f, s2 = 0.0f, s3 = 0.0f;
        int c = 0;
        for (; c + 3 < nparts; c += 4) {
            s0 += src[(int64_t)(c + 0) * step];
            s1 += src[(int64_t)(c + 1) * step];
            s2 += src[(int64_t)(c + 2) * step];
            s3 += src[(int64_t)(c + 3) * step];
        }
        for (; c < nparts; ++c) s0 += src[(int64_t)c * step];
        dW[(int64_t)n * ldw + k] = (s0 + s1) + (s2 + s3);
    }
}

// W[N,K] (row stride ldb) -> hi / lo pieces with row stride ldw.
__global__ void split_weight_kernel(const float *__restrict__ W, int64_t ldb, int N, int K, int ldw,
                                    float *__restrict__ hi, float *__restrict__ lo) {
    const int64_t total = (int64_t)N * ldw;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        const int n = (int)(i / ldw), k = (int)(i % ldw);
        float h = 0.0f, l = 0.0f;
        if (k < K) split_tf32(W[(int64_t)n * ldb + k], h, l);
        hi[i] = h;
        lo[i] = l;
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    });
    return fn;
}

// 2-D fp32 tensor map: `cols` contiguous elements per row, `rows` rows of stride ld elements;
// box = {box_cols, box_rows} with box_cols * 4 bytes = the swizzle span; out-of-range elements read
// as zero and are not written.
int make_map(CUtensorMap *map, const float *base, int64_t rows, int64_t cols, int64_t ld, int box_cols, int box_rows,
             int swizzle = -1) {
    EncodeTiledFn fn = encode_fn();
    if (fn == nullptr) return fail(GNNAGG_ERR_CUDA, "dense: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)ld * 4};
    const cuuint32_t box[2] = {(cuuint32_t)box_cols, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUtensorMapSwizzle swz = swizzle >= 0 ? (CUtensorMapSwizzle)swizzle
                                   : (box_cols == 32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, swz, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GNNAGG_ERR_CUDA, "dense: cuTensorMapEncodeTiled failed with code %d", (int)r);
    return GNNAGG_OK;
}

// Stall test: the launches that follow announce `tx_excess` bytes that never arrive, so their first wait for a
// load runs out after `wait_ns` and the kernel takes its abort path.  Zero in normal operation.
struct StallTest {
    unsigned long long wait_ns = kWaitLimitNs;
    uint32_t tx_excess = 0;
};
StallTest g_stall;

inline int round_up(int v, int m) { return (v + m - 1) / m * m; }
inline size_t piece_bytes(int N, int K) { return ((size_t)N * round_up(K, 4) * 4 + 255) / 256 * 256; }

}  // namespace
}  // namespace gnnagg

using namespace gnnagg;

extern "C" size_t gnnagg_dense_workspace_bytes(int32_t N, int32_t K) {
    if (N <= 0 || K <= 0) return kStatusBytes;
    return kStatusBytes + 2 * piece_bytes(N, K);
}

extern "C" int gnnagg_dense_tf32x3_f32(const float *A, int64_t lda, const float *B, int64_t ldb, float *C, int64_t ldc,
                                       int64_t M, int32_t N, int32_t K, const float *bias, int32_t accumulate,
                                       void *workspace, size_t workspace_bytes, void *stream) {
    if (M < 0 || N < 0 || K < 0 || (accumulate != 0 && accumulate != 1))
        return fail(GNNAGG_ERR_ARG, "dense: negative size or bad accumulate flag");
    if (M == 0 || N == 0) return GNNAGG_OK;
    if (A == nullptr || B == nullptr || C == nullptr || workspace == nullptr)
        return fail(GNNAGG_ERR_ARG, "dense: null pointer");
    if (K == 0) return fail(GNNAGG_ERR_UNSUPPORTED, "dense: K = 0");
    if (N > kMaxN) return fail(GNNAGG_ERR_UNSUPPORTED, "dense: N = %d exceeds %d output columns", N, kMaxN);
    if (lda < K || ldb < K || ldc < N) return fail(GNNAGG_ERR_ARG, "dense: leading dimension smaller than the row");
    if (!aligned16(A) || (lda % 4) != 0)
        return fail(GNNAGG_ERR_UNSUPPORTED, "dense: A must be 16-byte aligned with a row stride that is a multiple of 4");
    if (M > (int64_t)INT32_MAX - BM) return fail(GNNAGG_ERR_UNSUPPORTED, "dense: M too large for 32-bit tile coordinates");
    if (!aligned16(workspace) || workspace_bytes < gnnagg_dense_workspace_bytes(N, K))
        return fail(GNNAGG_ERR_SCRATCH, "dense: workspace too small or misaligned (need %zu bytes)",
                    gnnagg_dense_workspace_bytes(N, K));
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    const int ldw = round_up(K, 4);
    const int n_pad = round_up(N, 16);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    float *w_hi = reinterpret_cast<float *>(ws + kStatusBytes);
    float *w_lo = reinterpret_cast<float *>(ws + kStatusBytes + piece_bytes(N, K));

    static PerDeviceOnce attr_done;
    const cudaError_t attr_err = attr_done.run([] {
        return cudaFuncSetAttribute(gemm_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    });
    if (attr_err != cudaSuccess)
        return fail(GNNAGG_ERR_CUDA, "dense: cannot reserve %d bytes of shared memory: %s", SMEM_BYTES,
                    cudaGetErrorString(attr_err));

    // C goes out through TMA when its rows are 16-byte addressable, else through plain stores
    const bool tma_store = aligned16(C) && (ldc % 4) == 0;
    CUtensorMap map_a, map_bhi, map_blo, map_c;
    int rc = make_map(&map_a, A, M, K, lda, BK, BM);
    const int b_box_rows = n_pad;  // all weight rows of a k-block in one box (rows past N read as zero)
    if (rc == GNNAGG_OK) rc = make_map(&map_bhi, w_hi, N, K, ldw, BK, b_box_rows);
    if (rc == GNNAGG_OK) rc = make_map(&map_blo, w_lo, N, K, ldw, BK, b_box_rows);
    if (rc == GNNAGG_OK) {
        if (tma_store)
            rc = make_map(&map_c, C, M, N, ldc, 32, 32);
        else
            map_c = map_a;  // unused
    }
    if (rc != GNNAGG_OK) return rc;

    {
        const int64_t total = (int64_t)N * ldw;
        const unsigned blocks = (unsigned)((total + 255) / 256 > 1024 ? 1024 : (total + 255) / 256);
        split_weight_kernel<<<blocks, 256, 0, st>>>(B, ldb, N, K, ldw, w_hi, w_lo);
        rc = check_launch("split_weight_kernel");
        if (rc != GNNAGG_OK) return rc;
    }

    GemmParams p;
    p.C = C;
    p.bias = bias;
    p.status = reinterpret_cast<int *>(ws);
    p.M = M;
    p.ldc = ldc;
    p.N = N;
    p.n_pad = n_pad;
    p.K = K;
    p.accumulate = accumulate;
    p.num_tiles = (int)((M + BM - 1) / BM);
    p.tma_store = tma_store ? 1 : 0;
    p.b_box_rows = b_box_rows;
    p.wait_ns = g_stall.wait_ns;
    p.tx_excess = g_stall.tx_excess;
    const int grid = p.num_tiles < kNumSMs ? p.num_tiles : kNumSMs;
    gemm_tf32x3_kernel<<<grid, kThreads, SMEM_BYTES, st>>>(map_a, map_bhi, map_blo, map_c, p);
    return check_launch("gemm_tf32x3_kernel");
}


extern "C" size_t gnnagg_dense_wgrad_workspace_bytes(int32_t N, int32_t K) {
    if (N <= 0 || K <= 0) return kStatusBytes;
    return kStatusBytes + (size_t)kNumSMs * (size_t)N * (size_t)round_up(K, 4) * sizeof(float);
}

extern "C" int gnnagg_dense_wgrad_tf32x3_f32(const float *G, int64_t ldg, const float *X, int64_t ldx, int64_t M,
                                             int32_t N, int32_t K, float *dW, int64_t ldw, void *workspace,
                                             size_t workspace_bytes, void *stream) {
    if (M < 0 || N < 0 || K < 0) return fail(GNNAGG_ERR_ARG, "dense_wgrad: negative size");
    if (N == 0 || K == 0) return GNNAGG_OK;
    if (G == nullptr || X == nullptr || dW == nullptr || workspace == nullptr)
        return fail(GNNAGG_ERR_ARG, "dense_wgrad: null pointer");
    if (N > kMaxN || K > kMaxN)
        return fail(GNNAGG_ERR_UNSUPPORTED, "dense_wgrad: %d x %d exceeds %d x %d", N, K, kMaxN, kMaxN);
    if (ldg < N || ldx < K || ldw < K) return fail(GNNAGG_ERR_ARG, "dense_wgrad: leading dimension smaller than the row");
    if (!aligned16(G) || !aligned16(X) || (ldg % 4) != 0 || (ldx % 4) != 0)
        return fail(GNNAGG_ERR_UNSUPPORTED, "dense_wgrad: operands must be 16-byte aligned with row strides multiple of 4");
    if (M > (int64_t)INT32_MAX - WG_ROWS) return fail(GNNAGG_ERR_UNSUPPORTED, "dense_wgrad: M too large");
    if (!aligned16(workspace) || workspace_bytes < gnnagg_dense_wgrad_workspace_bytes(N, K))
        return fail(GNNAGG_ERR_SCRATCH, "dense_wgrad: workspace too small or misaligned (need %zu bytes)",
                    gnnagg_dense_wgrad_workspace_bytes(N, K));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    uint8_t *ws = static_cast<uint8_t *>(workspace);
    float *partial = reinterpret_cast<float *>(ws + kStatusBytes);
    if (M == 0) {
        for (int n = 0; n < N; ++n) {
            const cudaError_t e = cudaMemsetAsync(dW + (int64_t)n * ldw, 0, (size_t)K * 4, st);
            if (e != cudaSuccess) return fail(GNNAGG_ERR_CUDA, "dense_wgrad: %s", cudaGetErrorString(e));
        }
        return GNNAGG_OK;
    }

    static PerDeviceOnce attr_done;
    const cudaError_t attr_err = attr_done.run([] {
        return cudaFuncSetAttribute(wgrad_tf32x3_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, WG_SMEM_BYTES);
    });
    if (attr_err != cudaSuccess)
        return fail(GNNAGG_ERR_CUDA, "dense_wgrad: cannot reserve %d bytes of shared memory: %s", WG_SMEM_BYTES,
                    cudaGetErrorString(attr_err));

    // 32-bit MN-major operands use the 128-byte swizzle with 32-byte atoms, in the tensor map and in the
    // shared-memory descriptor (layout type 1); groups of 4 k-rows lie 512 bytes apart, boxes 2 KB apart
    const int swz = (int)CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B;
    CUtensorMap map_g, map_x;
    int rc = make_map(&map_g, G, M, N, ldg, 32, WG_ROWS, swz);
    if (rc == GNNAGG_OK) rc = make_map(&map_x, X, M, K, ldx, 32, WG_ROWS, swz);
    if (rc != GNNAGG_OK) return rc;

    WgradParams p;
    p.partial = partial;
    p.status = reinterpret_cast<int *>(ws);
    p.M = M;
    p.N = N;
    p.K = K;
    p.n_pad = round_up(K, 16);
    p.kp = round_up(K, 4);
    p.total_blocks = (int)((M + WG_ROWS - 1) / WG_ROWS);
    p.blocks_per_cta = (p.total_blocks + kNumSMs - 1) / kNumSMs;
    p.desc = smem_desc_mn_template(WG_BOX_BYTES, 512, 1);
    p.wait_ns = g_stall.wait_ns;
    p.tx_excess = g_stall.tx_excess;
    const int grid = (p.total_blocks + p.blocks_per_cta - 1) / p.blocks_per_cta;
    wgrad_tf32x3_kernel<<<grid, WG_THREADS, WG_SMEM_BYTES, st>>>(map_g, map_x, p);
    rc = check_launch("wgrad_tf32x3_kernel");
    if (rc != GNNAGG_OK) return rc;
    const int total = N * K;
    wgrad_reduce_kernel<<<(total + 255) / 256, 256, 0, st>>>(partial, grid, N, K, p.kp, dW, ldw);
    return check_launch("wgrad_reduce_kernel");
}

extern "C" int gnnagg_dense_status(const void *workspace, void *stream) {
    if (workspace == nullptr) return fail(GNNAGG_ERR_ARG, "dense_status: null workspace");
    int code = 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(&code, workspace, sizeof(int), cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess) return fail(GNNAGG_ERR_CUDA, "dense_status: %s", cudaGetErrorString(e));
    return code;
}

extern "C" int gnnagg_dense_status_clear(void *workspace, void *stream) {
    if (workspace == nullptr) return fail(GNNAGG_ERR_ARG, "dense_status_clear: null workspace");
    const cudaError_t e = cudaMemsetAsync(workspace, 0, sizeof(int), static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(GNNAGG_ERR_CUDA, "dense_status_clear: %s", cudaGetErrorString(e));
    return GNNAGG_OK;
}

extern "C" int gnnagg_dense_stall_test(int32_t tx_excess_bytes, int64_t wait_limit_us) {
    if (tx_excess_bytes < 0 || tx_excess_bytes > 1024 || wait_limit_us < 0 || wait_limit_us > 1000000)
        return fail(GNNAGG_ERR_ARG, "dense_stall_test: excess must be 0..1024 bytes, the limit 0..1e6 microseconds");
    g_stall.tx_excess = (uint32_t)tx_excess_bytes;
    g_stall.wait_ns = wait_limit_us == 0 ? kWaitLimitNs : (unsigned long long)wait_limit_us * 1000ull;
    return GNNAGG_OK;
}
