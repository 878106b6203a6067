// Halo exchange by direct stores: rows are written straight into the RECEIVING GPU's buffer over
// NVLink (plain st.global to peer-mapped memory), optionally gathered on the way, so the send-side
// staging buffer and the library all-to-all disappear.  One launch serves a group of peers:
// destination peer p gets this rank's block seg[p]..seg[p+1] at dst[p], the address inside p's
// receive buffer where this rank's rows belong.
//
// The kernel only stores to peer memory; it never loads from it, never waits on anything and uses no
// multicast of any kind.  Ordering with the consumer is the caller's: the receiving rank may read
// the rows after this kernel has completed and a collective ordered behind it (the caller uses a
// small NCCL all-reduce) has been seen on the receiver.
#include "common.cuh"

namespace gnnagg {

// Stores to a peer wait for NVLink; while they wait they hold the SM's path to the memory system, and every
// other warp of that SM waits with them (measured: with store CTAs on all SMs the SpMM on the compute
// stream made no progress until the exchange was over).  The exchange therefore runs on a FEW SMs, with
// large CTAs that keep them to themselves, like the channels of a collective library; the rest of the GPU
// belongs to the SpMM.  24 CTAs x 1024 threads x four rows in flight per lane group is several MB in
// flight, far more than NVLink's bandwidth-delay product.
constexpr int kPushCTAs = 24;
constexpr int kPushThreads = 1024;

// UNIT bytes per lane access (16 / 4 / 1); `units` of them per row; G = 2^log2g lanes per row.
template <typename T>
__global__ void __launch_bounds__(kPushThreads)
    push_rows_kernel(const uint8_t *__restrict__ src, int64_t ld_src, const int32_t *__restrict__ idx, int units,
                     int log2g, const int32_t *__restrict__ seg, int P, int first_peer, int num_peers,
                     const uint64_t *__restrict__ dst, int64_t ld_dst) {
    __shared__ int spre[kMaxSeg + 1];  // row prefix over the selected peers, in the order they are served
    if (threadIdx.x == 0) {
        int run = 0;
        for (int j = 0; j < num_peers; ++j) {
            int p = first_peer + j;
            if (p >= P) p -= P;
            spre[j] = run;
            run += seg[p + 1] - seg[p];
        }
        spre[num_peers] = run;
    }
    __syncthreads();
    const int total = spre[num_peers];
    const int G = 1 << log2g;
    const int gl = threadIdx.x & (G - 1);
    const int64_t groups_per_block = blockDim.x >> log2g;
    const int64_t stride = groups_per_block * gridDim.x;
    const int64_t first = (int64_t)blockIdx.x * groups_per_block + (threadIdx.x >> log2g);

    // send-list row v of the served peers -> where it is read and where it goes
    auto locate = [&](int64_t v, const T *&in, T *&out) {
        int lo = 0, hi = num_peers - 1;  // peer slot j with spre[j] <= v < spre[j+1] (empty peers skipped)
        while (lo < hi) {
            const int mid = (lo + hi + 1) >> 1;
            if (spre[mid] <= v)
                lo = mid;
            else
                hi = mid - 1;
        }
        int p = first_peer + lo;
        if (p >= P) p -= P;
        const int64_t r = v - spre[lo];          // row inside this rank's block for peer p
        const int64_t i = (int64_t)seg[p] + r;   // row of the send list
        const int64_t s = idx ? (int64_t)idx[i] : i;
        in = reinterpret_cast<const T *>(src + s * ld_src);
        out = reinterpret_cast<T *>(reinterpret_cast<uint8_t *>(dst[p]) + r * ld_dst);
    };

    if (units <= 2 * G) {
        // The grid is kept small (the SpMM running beside this kernel needs the SMs), so every lane keeps
        // several rows in flight: the loads of four rows are issued before the first store.
        constexpr int ROWS = 4;
        for (int64_t v0 = first; v0 < total; v0 += ROWS * stride) {
            T a[ROWS][2];
            T *out[ROWS];
#pragma unroll
            for (int q = 0; q < ROWS; ++q) {
                const int64_t v = v0 + q * stride;
                out[q] = nullptr;
                if (v < total) {
                    const T *in;
                    locate(v, in, out[q]);
                    if (gl < units) a[q][0] = __ldg(in + gl);
                    if (gl + G < units) a[q][1] = __ldg(in + gl + G);
                }
            }
#pragma unroll
            for (int q = 0; q < ROWS; ++q) {
                if (out[q] != nullptr) {
                    if (gl < units) out[q][gl] = a[q][0];
                    if (gl + G < units) out[q][gl + G] = a[q][1];
                }
            }
        }
    } else {
        for (int64_t v = first; v < total; v += stride) {
            const T *in;
            T *out;
            locate(v, in, out);
            for (int u = gl; u < units; u += G) out[u] = __ldg(in + u);
        }
    }
}

}  // namespace gnnagg

using namespace gnnagg;

extern "C" int gnnagg_push_rows(const void *src, int64_t ld_src, const int32_t *idx, int32_t row_bytes,
                                const int32_t *seg, int32_t P, int32_t first_peer, int32_t num_peers,
                                const uint64_t *dst, int64_t ld_dst, int64_t rows_hint, void *stream) {
    if (row_bytes < 0 || rows_hint < 0 || P < 1 || num_peers < 0 || num_peers > P || first_peer < 0 || first_peer >= P)
        return fail(GNNAGG_ERR_ARG, "push_rows: bad size or peer range");
    if (P > kMaxSeg) return fail(GNNAGG_ERR_UNSUPPORTED, "push_rows: more than %d peers", kMaxSeg);
    if (rows_hint == 0 || row_bytes == 0 || num_peers == 0) return GNNAGG_OK;
    if (src == nullptr || seg == nullptr || dst == nullptr || ld_src < row_bytes || ld_dst < row_bytes)
        return fail(GNNAGG_ERR_ARG, "push_rows: null pointer or leading dimension smaller than the row");
    // widest access both sides allow; the destination bases are checked by the caller (they are device data)
    int unit = 1;
    if (row_bytes % 16 == 0 && ld_src % 16 == 0 && ld_dst % 16 == 0 && aligned16(src)) unit = 16;
    else if (row_bytes % 4 == 0 && ld_src % 4 == 0 && ld_dst % 4 == 0 && (reinterpret_cast<uintptr_t>(src) & 3u) == 0) unit = 4;
    const int units = row_bytes / unit;
    int log2g = 0;
    while ((1 << log2g) < units && log2g < 5) ++log2g;
    const int64_t groups_per_block = kPushThreads >> log2g;
    int64_t blocks = div_up(rows_hint, groups_per_block * 4);
    if (blocks > kPushCTAs) blocks = kPushCTAs;
    if (blocks < 1) blocks = 1;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uint8_t *s8 = static_cast<const uint8_t *>(src);
#define GNNAGG_PUSH(T) \
    push_rows_kernel<T><<<(unsigned)blocks, kPushThreads, 0, st>>>(s8, ld_src, idx, units, log2g, seg, P, first_peer, num_peers, dst, ld_dst)
    if (unit == 16) GNNAGG_PUSH(uint4);
    else if (unit == 4) GNNAGG_PUSH(uint32_t);
    else GNNAGG_PUSH(uint8_t);
#undef GNNAGG_PUSH
    return check_launch("push_rows_kernel");
}

// One peer's block as ONE asynchronous device-to-device copy: the driver runs it on a copy engine, so the
// block crosses NVLink without occupying an SM (the store kernel above keeps 24 SMs busy for the length
// of the exchange).  For blocks that are contiguous on both sides -- everything but the forward fp32 halo
// of the plain plan, whose rows must be gathered first.
extern "C" int gnnagg_push_block(const void *src, void *dst, size_t bytes, void *stream) {
    if (bytes == 0) return GNNAGG_OK;
    if (src == nullptr || dst == nullptr) return fail(GNNAGG_ERR_ARG, "push_block: null pointer");
    const cudaError_t e = cudaMemcpyAsync(dst, src, bytes, cudaMemcpyDeviceToDevice, static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return fail(GNNAGG_ERR_CUDA, "push_block: %s", cudaGetErrorString(e));
    return GNNAGG_OK;
}
