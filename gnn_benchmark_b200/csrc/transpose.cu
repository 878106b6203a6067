// CSR -> CSC on the device: the operand of the transposed product (A^T G in backward), built once per
// matrix.  The reference gets it from its sparse-tensor package (colptr / row_T / value_T, cached on the
// matrix: model/ops/spmm_kernel.py:76-80); a torch.sort would do, at the price of three nnz-sized 64-bit
// temporaries.  Here it is a stable least-significant-digit radix sort of the nonzeros by column index
// (8-bit digits, only as many passes as the column count needs) that carries each nonzero's position:
//   pass  = per-tile digit histogram -> exclusive scan over (digit, tile) -> stable scatter;
//   tile  = 2048 consecutive elements owned by ONE warp, which ranks them 32 at a time with
//           __match_any_sync, so the order inside a digit is the input order without any sorting network;
//   end   = row_T[i] = row of nonzero perm[i] (binary search in rowptr), value_T[i] = val[perm[i]],
//           colptr = scan of the column histogram.
// CSR order has rows ascending, and the sort is stable: rows ascend inside every column, duplicates keep
// their order.  Everything is integer work on 32-bit keys: results are exact and run-to-run identical.
#include "common.cuh"

namespace gnnagg {

constexpr int kTileElems = 2048;   // per warp
constexpr int kSortWarps = 4;      // per CTA
constexpr int kScanBlock = 256;
constexpr int kScanPerThread = 8;  // 2048 elements per scan block

// ---- exclusive scan of int32 counts (out may be int32 in place, or int64) -----------------------------
template <typename OUT>
__global__ void __launch_bounds__(kScanBlock)
    scan_blocks_kernel(const int32_t *in, OUT *out, int64_t n, int64_t *__restrict__ block_sums) {  // out may be in
    __shared__ int64_t warp_tot[kScanBlock / 32];
    const int64_t base = ((int64_t)blockIdx.x * kScanBlock + threadIdx.x) * kScanPerThread;
    int64_t v[kScanPerThread];
    int64_t run = 0;
#pragma unroll
    for (int i = 0; i < kScanPerThread; ++i) {
        const int64_t x = (base + i < n) ? (int64_t)in[base + i] : 0;
        v[i] = run;
        run += x;
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int64_t incl = run;
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
        const int64_t t = __shfl_up_sync(kFullMask, incl, off);
        if (lane >= off) incl += t;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int64_t woff = 0;
    for (int w = 0; w < warp; ++w) woff += warp_tot[w];
    const int64_t toff = woff + incl - run;
#pragma unroll
    for (int i = 0; i < kScanPerThread; ++i)
        if (base + i < n) out[base + i] = (OUT)(toff + v[i]);
    if (threadIdx.x == kScanBlock - 1) block_sums[blockIdx.x] = toff + run;
}

// one CTA: exclusive scan of the block totals, in place; total -> block_sums[nb]
__global__ void __launch_bounds__(1024) scan_block_sums_kernel(int64_t *block_sums, int64_t nb) {
    __shared__ int64_t warp_tot[32];
    __shared__ int64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int64_t b0 = 0; b0 < nb; b0 += 1024) {
        const int64_t i = b0 + threadIdx.x;
        const int64_t x = i < nb ? block_sums[i] : 0;
        int64_t incl = x;
#pragma unroll
        for (int off = 1; off < 32; off <<= 1) {
            const int64_t t = __shfl_up_sync(kFullMask, incl, off);
            if (lane >= off) incl += t;
        }
        if (lane == 31) warp_tot[warp] = incl;
        __syncthreads();
        int64_t woff = 0;
        for (int w = 0; w < warp; ++w) woff += warp_tot[w];
        const int64_t c = carry;
        if (i < nb) block_sums[i] = c + woff + incl - x;
        __syncthreads();
        if (threadIdx.x == 1023) carry = c + woff + incl;
        __syncthreads();
    }
    if (threadIdx.x == 0) block_sums[nb] = carry;
}

template <typename OUT>
__global__ void __launch_bounds__(kScanBlock)
    scan_add_kernel(OUT *__restrict__ out, int64_t n, const int64_t *__restrict__ block_sums, OUT *total_at) {
    const int64_t base = ((int64_t)blockIdx.x * kScanBlock + threadIdx.x) * kScanPerThread;
    const int64_t off = block_sums[blockIdx.x];
#pragma unroll
    for (int i = 0; i < kScanPerThread; ++i)
        if (base + i < n) out[base + i] += (OUT)off;
    if (total_at != nullptr && blockIdx.x == 0 && threadIdx.x == 0) *total_at = (OUT)block_sums[gridDim.x];
}

template <typename OUT>
static int exclusive_scan(const int32_t *in, OUT *out, int64_t n, int64_t *block_sums, OUT *total_at, cudaStream_t st) {
    const int64_t nb = div_up(n, (int64_t)kScanBlock * kScanPerThread);
    scan_blocks_kernel<OUT><<<(unsigned)nb, kScanBlock, 0, st>>>(in, out, n, block_sums);
    scan_block_sums_kernel<<<1, 1024, 0, st>>>(block_sums, nb);
    scan_add_kernel<OUT><<<(unsigned)nb, kScanBlock, 0, st>>>(out, n, block_sums, total_at);
    return check_launch("scan kernels");
}

// ---- radix pass ----------------------------------------------------------------------------------------
__global__ void iota_kernel(int32_t *__restrict__ p, int64_t n) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = (int32_t)i;
}

__global__ void column_histogram_kernel(const int32_t *__restrict__ col, int64_t nnz, int32_t *__restrict__ cnt) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; e < nnz; e += stride) atomicAdd(cnt + col[e], 1);
}

// hist[digit * ntiles + tile] = number of keys of the tile with that digit
__global__ void __launch_bounds__(kSortWarps * 32)
    radix_hist_kernel(const int32_t *__restrict__ keys, int64_t n, int shift, int64_t ntiles, int32_t *__restrict__ hist) {
    __shared__ int cnt[kSortWarps][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tile = (int64_t)blockIdx.x * kSortWarps + warp;
    for (int d = lane; d < 256; d += 32) cnt[warp][d] = 0;
    __syncwarp();
    if (tile < ntiles) {
        const int64_t base = tile * kTileElems;
        for (int r = 0; r < kTileElems / 32; ++r) {
            const int64_t i = base + r * 32 + lane;
            const bool ok = i < n;
            const int d = ok ? ((keys[i] >> shift) & 255) : 256 + lane;  // out-of-range lanes match nobody
            const unsigned peers = __match_any_sync(kFullMask, d);
            if (ok && lane == (__ffs(peers) - 1)) cnt[warp][d] += __popc(peers);
            __syncwarp();
        }
        for (int d = lane; d < 256; d += 32) hist[(int64_t)d * ntiles + tile] = cnt[warp][d];
    }
}

// offs = exclusive scan of hist; element i of the tile goes to offs[digit][tile] + (number of earlier
// elements of the tile with the same digit)
__global__ void __launch_bounds__(kSortWarps * 32)
    radix_scatter_kernel(const int32_t *__restrict__ keys, const int32_t *__restrict__ pay, int64_t n, int shift,
                         int64_t ntiles, const int32_t *__restrict__ offs, int32_t *__restrict__ keys_out,
                         int32_t *__restrict__ pay_out) {
    __shared__ int pos[kSortWarps][256];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t tile = (int64_t)blockIdx.x * kSortWarps + warp;
    if (tile >= ntiles) return;
    for (int d = lane; d < 256; d += 32) pos[warp][d] = offs[(int64_t)d * ntiles + tile];
    __syncwarp();
    const int64_t base = tile * kTileElems;
    const unsigned lt = (1u << lane) - 1u;
    for (int r = 0; r < kTileElems / 32; ++r) {
        const int64_t i = base + r * 32 + lane;
        const bool ok = i < n;
        int k = 0, p = 0;
        if (ok) {
            k = keys[i];
            p = pay[i];
        }
        const int d = ok ? ((k >> shift) & 255) : 256 + lane;
        const unsigned peers = __match_any_sync(kFullMask, d);
        int dst = 0;
        if (ok) dst = pos[warp][d] + __popc(peers & lt);
        __syncwarp();
        if (ok && lane == (__ffs(peers) - 1)) pos[warp][d] += __popc(peers);
        __syncwarp();
        if (ok) {
            keys_out[dst] = k;
            pay_out[dst] = p;
        }
    }
}

__global__ void csc_finish_kernel(const int64_t *__restrict__ rowptr, int64_t M, const float *__restrict__ val,
                                  const int32_t *__restrict__ perm, int64_t nnz, int32_t *__restrict__ row_T,
                                  float *__restrict__ val_T) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < nnz; i += stride) {
        const int64_t e = perm[i];
        int64_t lo = 0, hi = M - 1;  // last row with rowptr[row] <= e
        while (lo < hi) {
            const int64_t mid = (lo + hi + 1) >> 1;
            if (rowptr[mid] <= e)
                lo = mid;
            else
                hi = mid - 1;
        }
        row_T[i] = (int32_t)lo;
        val_T[i] = val[e];
    }
}

struct TransposeLayout {
    size_t keys_a, keys_b, pay_a, pay_b, hist, block_sums, cnt, total;
};

static TransposeLayout transpose_layout(int64_t K, int64_t nnz) {
    auto up = [](size_t x) { return (x + 255) & ~(size_t)255; };
    const int64_t ntiles = div_up(nnz, kTileElems);
    const int64_t hist_n = 256 * (ntiles > 0 ? ntiles : 1);
    const int64_t scan_n = hist_n > K + 1 ? hist_n : K + 1;
    TransposeLayout l;
    size_t off = 0;
    l.keys_a = off, off += up((size_t)nnz * 4);
    l.keys_b = off, off += up((size_t)nnz * 4);
    l.pay_a = off, off += up((size_t)nnz * 4);
    l.pay_b = off, off += up((size_t)nnz * 4);
    l.hist = off, off += up((size_t)hist_n * 4);
    l.block_sums = off, off += up((size_t)(div_up(scan_n, (int64_t)kScanBlock * kScanPerThread) + 2) * 8);
    l.cnt = off, off += up((size_t)(K + 1) * 4);
    l.total = off;
    return l;
}

}  // namespace gnnagg

using namespace gnnagg;

extern "C" size_t gnnagg_csr_to_csc_workspace_bytes(int64_t M, int64_t K, int64_t nnz) {
    if (M < 0 || K < 0 || nnz < 0) return 0;
    return transpose_layout(K, nnz).total;
}

extern "C" int gnnagg_csr_to_csc(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                                 int64_t nnz, int64_t *colptr, int32_t *row_T, float *val_T, void *workspace,
                                 size_t workspace_bytes, void *stream) {
    if (M < 0 || K < 0 || nnz < 0) return fail(GNNAGG_ERR_ARG, "csr_to_csc: negative size");
    if (colptr == nullptr || rowptr == nullptr) return fail(GNNAGG_ERR_ARG, "csr_to_csc: null pointer");
    if (M > INT32_MAX || K > INT32_MAX - 1 || nnz > INT32_MAX)
        return fail(GNNAGG_ERR_UNSUPPORTED, "csr_to_csc: M, K and nnz must fit int32");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (nnz == 0) {
        const cudaError_t e = cudaMemsetAsync(colptr, 0, (size_t)(K + 1) * 8, st);
        return e == cudaSuccess ? GNNAGG_OK : fail(GNNAGG_ERR_CUDA, "csr_to_csc: %s", cudaGetErrorString(e));
    }
    if (col == nullptr || val == nullptr || row_T == nullptr || val_T == nullptr)
        return fail(GNNAGG_ERR_ARG, "csr_to_csc: null pointer");
    const TransposeLayout l = transpose_layout(K, nnz);
    if (workspace == nullptr || workspace_bytes < l.total || (reinterpret_cast<uintptr_t>(workspace) & 255u))
        return fail(GNNAGG_ERR_SCRATCH, "csr_to_csc: workspace missing, smaller than %zu bytes or not 256-byte aligned", l.total);
    char *w = static_cast<char *>(workspace);
    int32_t *keys[2] = {reinterpret_cast<int32_t *>(w + l.keys_a), reinterpret_cast<int32_t *>(w + l.keys_b)};
    int32_t *pay[2] = {reinterpret_cast<int32_t *>(w + l.pay_a), reinterpret_cast<int32_t *>(w + l.pay_b)};
    int32_t *hist = reinterpret_cast<int32_t *>(w + l.hist);
    int64_t *block_sums = reinterpret_cast<int64_t *>(w + l.block_sums);
    int32_t *cnt = reinterpret_cast<int32_t *>(w + l.cnt);

    // colptr = exclusive scan of the column histogram (K+1 entries, the last one = nnz)
    cudaMemsetAsync(cnt, 0, (size_t)(K + 1) * 4, st);
    column_histogram_kernel<<<kNumSMs * 8, 256, 0, st>>>(col, nnz, cnt);
    int rc = exclusive_scan<int64_t>(cnt, colptr, K + 1, block_sums, nullptr, st);
    if (rc != GNNAGG_OK) return rc;

    // stable sort of (column, position) by column
    const int64_t ntiles = div_up(nnz, kTileElems);
    const unsigned tile_blocks = (unsigned)div_up(ntiles, kSortWarps);
    iota_kernel<<<(unsigned)div_up(nnz, 256), 256, 0, st>>>(pay[0], nnz);
    int bits = 1;
    while (bits < 31 && ((int64_t)1 << bits) < K) ++bits;
    const int32_t *kin = col;
    int cur = 0;
    for (int shift = 0; shift < bits; shift += 8) {
        radix_hist_kernel<<<tile_blocks, kSortWarps * 32, 0, st>>>(kin, nnz, shift, ntiles, hist);
        rc = exclusive_scan<int32_t>(hist, hist, 256 * ntiles, block_sums, nullptr, st);
        if (rc != GNNAGG_OK) return rc;
        radix_scatter_kernel<<<tile_blocks, kSortWarps * 32, 0, st>>>(kin, pay[cur], nnz, shift, ntiles, hist,
                                                                      keys[cur ^ 1], pay[cur ^ 1]);
        kin = keys[cur ^ 1];
        cur ^= 1;
    }
    csc_finish_kernel<<<kNumSMs * 8, 256, 0, st>>>(rowptr, M, val, pay[cur], nnz, row_T, val_T);
    return check_launch("csr_to_csc kernels");
}
