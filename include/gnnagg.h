/*
 * libgnnagg -- C ABI of the B200 (sm_100a) graph-aggregation kernels.
 *
 * This is the boundary a maintainer of the reference binds in place of its pybind11
 * module `computation_ops` (self_benchmark/a64fx/model/ops/src/ops.cpp:11-24).
 *
 * Conventions
 *   - every pointer is a DEVICE pointer owned by the caller unless its comment says
 *     "host"; nothing here allocates or frees device memory;
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised;
 *   - dense matrices are row-major fp32 with an explicit leading dimension in elements;
 *   - return value: 0 = ok, < 0 = argument / launch error found on the host
 *     (see gnnagg_error_string), never a device trap;
 *   - safe to call from one host thread per GPU; the library keeps no global state
 *     apart from a thread-local message for the last error and the built-in scratch
 *     buffer of gnnagg_spmm_csr_f32_static_scratch.
 */
#ifndef GNNAGG_H
#define GNNAGG_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define GNNAGG_OK 0
#define GNNAGG_ERR_ARG (-1)         /* null pointer, negative size, bad flag          */
#define GNNAGG_ERR_UNSUPPORTED (-2) /* shape outside what the kernels are built for   */
#define GNNAGG_ERR_CUDA (-3)        /* cudaGetLastError() after the launch was not ok */
#define GNNAGG_ERR_SCRATCH (-4)     /* plan / scratch buffer too small or malformed   */

/* Library version (major*10000 + minor*100 + patch). */
int gnnagg_version(void);

/* Static text for a status code; the thread's last detailed message when code < 0 and
 * one was recorded.  Never NULL. */
const char *gnnagg_error_string(int code);

/* ------------------------------------------------------------------------------------
 * K1  CSR SpMM   Y[M,F] (+)= A[M,K] * X[K,F]
 *
 * Replaces computation_ops.spmm == spmm_cpu_optimized_no_tile_v1
 * (model/ops/src/spmm.cpp:327-507, inner loop kernel_1xN :24-143) and the greedy
 * per-thread row split computed by distribute_work_for_row
 * (model/ops/spmm_kernel.py:7-28), which becomes the `plan` below.
 *
 * The transposed product (SPMM_backward, model/ops/spmm_kernel.py:71-90) is the same
 * call on the CSC arrays (colptr, row_T, value_T) with its own plan.
 *
 * A plan is an opaque, relocatable byte buffer describing how the (rows + nonzeros) of
 * one sparsity pattern are cut into equal work chunks (merge-path).  It depends only
 * on rowptr, is built once per matrix and is valid for every F.
 *
 * scratch: device buffer of gnnagg_spmm_scratch_bytes(); holds the partial sums of the
 * rows that are cut across chunks (hub rows).  Contents need not be initialised and are
 * garbage afterwards; two SpMM calls that may overlap on the GPU need separate scratch.
 *
 * accumulate != 0 : Y += A*X (the reference's semantics: it loads `out` first,
 *                   spmm.cpp:79-95);  accumulate == 0 : Y = A*X, empty rows written 0.
 * Summation order: nonzeros of a row are applied in CSR order with one fused
 * multiply-add each, as in the reference, whenever the row is processed by one
 * chunk and F > 64; rows cut across chunks, and narrower F (several nonzeros in
 * flight per warp), differ from it only by fp32 re-association.  The result is
 * deterministic (no float atomics).
 * ---------------------------------------------------------------------------------- */
size_t gnnagg_spmm_plan_bytes(int64_t M, int64_t nnz);
int gnnagg_spmm_plan_build(const int64_t *rowptr, int64_t M, int64_t nnz, void *plan, size_t plan_bytes,
                           void *stream);
size_t gnnagg_spmm_scratch_bytes(int64_t M, int64_t nnz, int32_t F);
int gnnagg_spmm_csr_f32(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                        int64_t nnz, const float *X, int64_t ldx, float *Y, int64_t ldy, int32_t F,
                        int32_t accumulate, const void *plan, void *scratch, size_t scratch_bytes,
                        void *stream);

/* CSR -> CSC: the operand of the transposed product (SPMM_backward), built once per matrix.  Replaces the
 * `src.storage.colptr() / row_T() / value_T()` arrays the reference takes from its sparse-tensor package
 * and caches on the matrix (model/ops/spmm_kernel.py:76-80).  Stable: rows ascend inside every column,
 * duplicated entries keep their CSR order.
 *   colptr int64[K+1], row_T int32[nnz], val_T fp32[nnz]: outputs;
 *   workspace: gnnagg_csr_to_csc_workspace_bytes(M, K, nnz) bytes, 256-byte aligned (about 16 bytes per
 *   nonzero: a stable 8-bit-digit radix sort of (column, position) pairs).  M, K, nnz < 2^31. */
size_t gnnagg_csr_to_csc_workspace_bytes(int64_t M, int64_t K, int64_t nnz);
int gnnagg_csr_to_csc(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K, int64_t nnz,
                      int64_t *colptr, int32_t *row_T, float *val_T, void *workspace, size_t workspace_bytes,
                      void *stream);

/* K3b + K4 fused: the same SpMM with the dense operand given as a row-packed quantised halo buffer
 * instead of fp32 rows.  Column index c of the sparse matrix is a wire slot; its feature row is
 * decoded on the fly as fma(code, scale_c, zero_point_c) with the bf16 wire parameters -- exactly
 * the value gnnagg_unpack_dequant_rows would have stored -- and enters the same FMA chain, so the
 * result equals unpack + gnnagg_spmm_csr_f32 bit for bit while the fp32 halo buffer is never
 * written or read (4F -> F*bits/8 + 4 gathered bytes per nonzero).
 * Replaces the pair dequantize_tensor_for_all_procs (quantization_arm.cpp:437-479) + spmm on the
 * receive side of the exchange (model/layers/aggregator.py:83-104, :180-199).
 *   codes / params_bf16 / seg / P / bits: as produced by gnnagg_quant_pack_rows on the sender and
 *   laid out by the receiver's own segment prefix; K = seg[P] wire slots.  F % 4 == 0 required. */
int gnnagg_spmm_csr_q(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                      int64_t nnz, const uint8_t *codes, const void *params_bf16, const int32_t *seg, int32_t P,
                      int32_t bits, float *Y, int64_t ldy, int32_t F, int32_t accumulate, const void *plan,
                      void *scratch, size_t scratch_bytes, void *stream);

/* Same product as gnnagg_spmm_csr_f32 for callers that cannot allocate device memory where they
 * call it (code under a host framework whose allocator may not be used at that point, a plugin
 * that is handed nothing but its operands, a process with a device-memory budget fixed up front):
 * the partial-sum scratch is a fixed buffer of GNNAGG_STATIC_SCRATCH_BYTES inside the library,
 * held by every GPU that loads the library until the process exits.  This entry point has no
 * counterpart in the reference.
 *   - Limit: gnnagg_spmm_scratch_bytes(M, nnz, F) must not exceed GNNAGG_STATIC_SCRATCH_BYTES
 *     (with the default chunking about 16 million rows+nonzeros at F = 256, 33 million at
 *     F <= 128); larger products return GNNAGG_ERR_SCRATCH and launch nothing.
 *   - It calls no cudaMalloc / cudaFree and no allocating routine; plan, operands and output
 *     still come from the caller.
 *   - The first call on each device looks up the buffer's address for that device (with that
 *     device current); make that first call before any stream capture begins.
 *   - All calls on a device share the one buffer, which keeps the previous call's contents.
 *     Nothing in it needs to start at zero (every slot that is read was written earlier in the
 *     same call), but two calls that may run on the GPU at the same time -- different streams,
 *     different host threads -- race on it: keep calls on one device in one stream order. */
#define GNNAGG_STATIC_SCRATCH_BYTES (32u << 20)
int gnnagg_spmm_csr_f32_static_scratch(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M,
                                       int64_t K, int64_t nnz, const float *X, int64_t ldx, float *Y, int64_t ldy,
                                       int32_t F, int32_t accumulate, const void *plan, void *stream);

/* Checks on the device that rowptr is monotone with rowptr[0]==0, rowptr[M]==nnz and
 * that every col is in [0,K).  status (device int32[1]) receives 0 or a bit mask
 * (1 = rowptr, 2 = col); the caller reads it back.  Has no counterpart in the
 * reference, which trusts its inputs; used by the host layer before a first launch. */
int gnnagg_csr_validate(const int64_t *rowptr, const int32_t *col, int64_t M, int64_t K, int64_t nnz,
                        int32_t *status, void *stream);

/* ------------------------------------------------------------------------------------
 * K2a  row gather   OUT[i,:] = X[idx[i],:]
 * Replaces torch.index_select(local_nodes_feat, 0, idx_nodes_send_to_others, out=send_buf)
 * (model/layers/aggregator.py:51).
 * ---------------------------------------------------------------------------------- */
int gnnagg_gather_rows_f32(const float *X, int64_t ldx, const int32_t *idx, int64_t rows, int32_t F,
                           float *OUT, int64_t ldo, void *stream);

/* Exchange by direct stores: rows of this rank's send list are written straight into the receiving
 * GPUs' buffers (peer-mapped memory, plain stores over NVLink), gathered on the way when idx != NULL.
 * Replaces the send-buffer fill and the all-to-all of the halo exchange for the peers it serves:
 *   torch.index_select(x, 0, idx_nodes_send_to_others, out=send_buf)   (model/layers/aggregator.py:51)
 *   dist.all_to_all_single(recv_buf, send_buf, recv_splits, send_splits) (communicator.py:101, :307-311)
 *   src        rows of row_bytes bytes, leading dimension ld_src bytes (fp32 rows: 4F; packed code rows:
 *              F; bf16 parameter pairs: 4)
 *   idx        optional int32 gather index: send-list row i is src row idx[i]; NULL = row i
 *   seg        device int32[P+1], prefix of the send list's per-peer row counts
 *   first_peer, num_peers: the peers served by this launch, first_peer, first_peer+1, ... (mod P)
 *   dst        device uint64[P]: dst[p] = address, valid on THIS device, of the place in peer p's receive
 *              buffer where this rank's block starts; rows land there with leading dimension ld_dst
 *              bytes.  Bases and leading dimensions must allow the access width the source allows
 *              (16 bytes when row_bytes, ld_src, ld_dst are multiples of 16 and src is 16-byte aligned).
 *   rows_hint  number of rows these peers get (host copy of the splits; sizes the grid)
 * The kernel stores to peer memory only: no loads from it, no waiting, no multicast.  The receiver may
 * read the rows once this launch has completed and it has been told so (e.g. by a collective queued
 * behind the launch). */
int gnnagg_push_rows(const void *src, int64_t ld_src, const int32_t *idx, int32_t row_bytes, const int32_t *seg,
                     int32_t P, int32_t first_peer, int32_t num_peers, const uint64_t *dst, int64_t ld_dst,
                     int64_t rows_hint, void *stream);
/* The same exchange for a block that is contiguous on both sides (the send buffer's rows for one peer,
 * packed codes, bf16 parameters): one asynchronous device-to-device copy of `bytes` bytes from src to
 * dst (an address inside the peer's receive buffer, valid on this device), queued on `stream`.  The
 * driver runs it on a copy engine: no SM is occupied while the block crosses NVLink.  Replaces the same
 * all_to_all_single message (communicator.py:101, :307-311). */
int gnnagg_push_block(const void *src, void *dst, size_t bytes, void *stream);

/* Y[i,:] = X[i,:] * s[i] (divide == 0) or X[i,:] / s[i] (divide == 1, IEEE quotient), plus bias[F] when
 * bias != NULL; Y may alias X.  Replaces the broadcast `out /= graph.in_degrees` of the layer
 * (model/layers/sageconv.py:84-85) and the d^-1/2 row scalings (and bias add) of a GCN layer around
 * the aggregation. */
int gnnagg_scale_rows_f32(const float *X, int64_t ldx, const float *s, int64_t rows, int32_t F, int32_t divide,
                          const float *bias, float *Y, int64_t ldy, void *stream);

/* ------------------------------------------------------------------------------------
 * K3a  per-row min/max quantise + row-pack, one call for all peer segments
 *
 * Replaces computation_ops.quantize_tensor_for_all_procs
 * (model/ops/src/quantization_arm.cpp:364-435, kernel :80-217, segmenting :21-78) for
 * bits == 2, and, with one segment, the row-packed layout of the x86
 * computation_ops.quantize_tensor (model/ops/src/quantization_x86.cpp:17-102) for
 * bits in {2,4,8}.
 *
 *   seg        device int32[P+1], prefix of per-peer row counts (seg[0] == 0)
 *   idx        optional: row i is read from X[idx[i],:] (fuses K2a); NULL = X[i,:]
 *   params     (rows,2) fp32 [zero_point, scale].  params_given == 0: computed here
 *              (zero_point = row min, scale = (max-min)/(2^bits-1), 0 -> 1) and written;
 *              params_given != 0: read (the x86 generic signature: caller-supplied).
 *   params_bf16 optional (rows,2) bf16 copy of params, round-to-nearest-even: the wire
 *              format of communicator.py:297 (fuses that cast); NULL to skip.
 *   codes      (sum_p ceil(n_p / (8/bits)), F) uint8, row stride F; 8/bits consecutive
 *              rows of one segment share a byte per column, first row in the high bits.
 * ---------------------------------------------------------------------------------- */
int gnnagg_quant_pack_rows(const float *X, int64_t ldx, const int32_t *idx, int32_t F, const int32_t *seg,
                           int32_t P, int64_t rows, int32_t bits, int32_t params_given, float *params,
                           void *params_bf16, uint8_t *codes, void *stream);

/* K2 + K3a fused: SpMM whose output rows are quantised + packed in its epilogue instead of stored.
 * Row i of the CSR matrix is wire slot i.  The kernel is gnnagg_spmm_csr_f32's (same plan, same chunking,
 * same summation order); where that one would store a finished row it encodes the row from the registers
 * that hold it and ORs its codes into the packed buffer, so the fp32 send buffer of the exchange is never
 * written or read.  Rows cut across chunks (hub vertices) are finished and encoded by the fix-up kernel.
 * Replaces the pair
 *   SPMM_forward(adj_t_pre_post_aggr_to, x, send_buf)            (model/layers/aggregator.py:48-49)
 *   quantize_tensor_for_all_procs(send_buf, ...)                 (communicator.py:281-284,
 *                                                                 model/ops/src/quantization_arm.cpp:364-435)
 * and, with the CSC arrays of the receive-side matrix as (rowptr, col, val), the backward pair
 *   SPMM_backward(remote_adj_t | adj_t_pre_post_aggr_from, grad, recv_buf) + quantise
 *                                                                (model/layers/aggregator.py:145-149).
 *   M = number of wire slots = seg[P];  X (K,F) fp32 with leading dimension ldx;
 *   params / params_bf16 / codes / seg / P / bits: as for gnnagg_quant_pack_rows (params computed here);
 *   plan: gnnagg_spmm_plan_build of this matrix; scratch: gnnagg_spmm_quant_pack_scratch_bytes(M, nnz, F).
 * Needs F % 4 == 0, F <= 512, ldx % 4 == 0 and 16-byte aligned X (GNNAGG_ERR_UNSUPPORTED otherwise: run
 * the two calls).  Codes and parameters are bit-identical to gnnagg_spmm_csr_f32(accumulate = 0) followed
 * by gnnagg_quant_pack_rows, for every width and row length. */
size_t gnnagg_spmm_quant_pack_scratch_bytes(int64_t M, int64_t nnz, int32_t F);
int gnnagg_spmm_quant_pack(const int64_t *rowptr, const int32_t *col, const float *val, int64_t M, int64_t K,
                           int64_t nnz, const float *X, int64_t ldx, int32_t F, const int32_t *seg, int32_t P,
                           int32_t bits, float *params, void *params_bf16, uint8_t *codes, const void *plan,
                           void *scratch, size_t scratch_bytes, void *stream);

/* ------------------------------------------------------------------------------------
 * K3b  unpack + dequantise   OUT[i,k] = fma(code, scale_i, zero_point_i)
 *
 * Replaces computation_ops.dequantize_tensor_for_all_procs
 * (model/ops/src/quantization_arm.cpp:437-479, kernel :219-299) and, with one segment,
 * the x86 dequantize_tensor (model/ops/src/quantization_x86.cpp:104-168; its
 * val*scale+min is one fma under the reference's own build flags).
 *
 *   params_bf16 != NULL: parameters are read from the bf16 wire buffer (fuses the
 *   bf16 -> fp32 copy of communicator.py:303) and, if params != NULL, the widened fp32
 *   values are also stored there; params_bf16 == NULL: parameters are read from params.
 * ---------------------------------------------------------------------------------- */
int gnnagg_unpack_dequant_rows(const uint8_t *codes, int32_t F, const int32_t *seg, int32_t P, int64_t rows,
                               int32_t bits, float *params, const void *params_bf16, float *OUT, int64_t ldo,
                               void *stream);

/* ------------------------------------------------------------------------------------
 * K3c  mixed-bit column-packed codec (per-row bits in {8,4,2})
 *
 * Replaces computation_ops.quantize_tensor_v1 / dequantize_tensor_v1
 * (model/ops/src/quantization_x86.cpp:170-312, quantization_kernel_x86.h:11-75).
 *   params (rows,3) fp32 [bits, zero_point, scale]; bits is read, the other two written
 *   (quantise) or read (dequantise).  range int64[rows+1]: byte offsets of each row in
 *   codes (quantizer.py:69-76).
 * ---------------------------------------------------------------------------------- */
int gnnagg_quant_v1_rows(const float *X, int64_t ldx, int64_t rows, int32_t F, const int64_t *range,
                         float *params, uint8_t *codes, void *stream);
int gnnagg_dequant_v1_rows(const uint8_t *codes, int64_t rows, int32_t F, const int64_t *range,
                           const float *params, float *OUT, int64_t ldo, void *stream);

/* fp32 <-> bf16 (round-to-nearest-even) buffer casts of the 16-bit halo mode
 * (communicator.py:128,137: send_buf_fp16.copy_(send_buf), recv_buf.copy_(recv_buf_fp16)). */
int gnnagg_cast_f32_to_bf16(const float *src, void *dst_bf16, int64_t n, void *stream);
int gnnagg_cast_bf16_to_f32(const void *src_bf16, float *dst, int64_t n, void *stream);

/* ------------------------------------------------------------------------------------
 * N1  dense feature transform on the tensor cores (the step either side of the aggregation)
 *
 *     C[M,N] (+)= A[M,K] . B[N,K]^T (+ bias[N])        fp32 in, fp32 out, row-major
 *
 * Replaces the fp32 nn.Linear calls of the layer around the aggregation op
 * (model/layers/sageconv.py:82-91: lin_neigh(out) + lin_self(x) + bias) and their input
 * gradients.  B is a Linear weight (out_features x in_features).  Every operand is split into two
 * TF32 pieces and three tcgen05 products are accumulated in fp32 (error about 2^-21 per product
 * relative to |a||b|: fp32-grade, not single-pass TF32).
 *
 *   N <= 256;  A 16-byte aligned with lda % 4 == 0 (TMA);  B, C, bias: any alignment.
 *   workspace  gnnagg_dense_workspace_bytes(N, K) bytes, 16-byte aligned, ZEROED once by the
 *              caller before its first use: the first 256 bytes hold a sticky status word, the
 *              rest receives the split weight (rewritten by every call).
 *   Calls sharing a workspace must be ordered on one stream.
 *
 * gnnagg_dense_status synchronises the stream and returns the status word: 0, or the positive
 * code of the wait that ran out of time inside the kernel (1 free stage, 2 TMA load, 3 split
 * tile, 4 accumulator release, 5 accumulator, 6 drain).  A kernel that gave up has freed its
 * tensor memory and returned; C is then undefined.
 * ---------------------------------------------------------------------------------- */
size_t gnnagg_dense_workspace_bytes(int32_t N, int32_t K);
int gnnagg_dense_tf32x3_f32(const float *A, int64_t lda, const float *B, int64_t ldb, float *C, int64_t ldc,
                            int64_t M, int32_t N, int32_t K, const float *bias, int32_t accumulate,
                            void *workspace, size_t workspace_bytes, void *stream);
int gnnagg_dense_status(const void *workspace, void *stream);
/* Resets the status word of a workspace to 0 (stream-ordered). */
int gnnagg_dense_status_clear(void *workspace, void *stream);
/* Test hook (no reference counterpart): while tx_excess_bytes > 0 the dense launches of this process
 * announce that many bytes more to their load barriers than their copies deliver, so the first wait for a
 * load runs out after wait_limit_us microseconds and the kernel takes its give-up path (status word set,
 * copies and MMAs drained, tensor memory freed, return).  (0, 0) restores normal operation and the normal
 * limit of one second.  Nothing faults or hangs: the copies themselves are unchanged and complete. */
int gnnagg_dense_stall_test(int32_t tx_excess_bytes, int64_t wait_limit_us);

/* Weight gradient of the same layer, dW[N,K] = G[M,N]^T . X[M,K] (overwritten), on the tensor cores
 * with the same three-product TF32 split; replaces the `grad_out.t() @ input` products of the
 * Linear layers' backward.  N, K <= 256; G and X 16-byte aligned with row strides % 4 == 0.
 * workspace: gnnagg_dense_wgrad_workspace_bytes(N, K) bytes, 16-byte aligned, zeroed once before
 * first use (status word as above, then one partial product per SM that a second kernel adds in a
 * fixed order). */
size_t gnnagg_dense_wgrad_workspace_bytes(int32_t N, int32_t K);
int gnnagg_dense_wgrad_tf32x3_f32(const float *G, int64_t ldg, const float *X, int64_t ldx, int64_t M, int32_t N,
                                  int32_t K, float *dW, int64_t ldw, void *workspace, size_t workspace_bytes,
                                  void *stream);

/* ------------------------------------------------------------------------------------
 * N1  dropout -> LayerNorm -> ReLU of the hidden layers, one pass forward, one backward
 *
 * Replaces F.dropout + LayerNorm + F.relu between the layers (model/DistSAGE.py:49-54) and
 * their three backward passes.  One warp per row; F % 4 == 0, F <= 1024, rows 16-byte aligned.
 *
 *   Y = relu(LN(D) * gamma + beta),  D = X * keep / (1 - p);  LN over the F columns, biased variance.
 *   keep: Philox-4x32-10 keyed by `seed`, counter (row, 4-column chunk); p is quantised to 1/65536.
 *   mask   rows * F/4 bytes, 4 keep-bits per chunk; written when p > 0 (needed by backward).
 *   stats  rows * 2 floats (mean, rstd) or NULL (inference: nothing kept for backward).
 * Backward reads GY and X once, rebuilds the normalised row and the ReLU decision with the
 * forward's arithmetic, writes GX, and leaves per-CTA column sums in `partial`
 * (gnnagg_dropout_ln_relu_partial_bytes(F) bytes) that a second kernel adds in a fixed order
 * into dgamma / dbeta (overwritten).
 * ---------------------------------------------------------------------------------- */
size_t gnnagg_dropout_ln_relu_partial_bytes(int32_t F);
int gnnagg_dropout_ln_relu_fwd(const float *X, int64_t ldx, int64_t rows, int32_t F, const float *gamma,
                               const float *beta, float eps, float p_drop, uint64_t seed, float *Y, int64_t ldy,
                               uint8_t *mask, float *stats, void *stream);
int gnnagg_dropout_ln_relu_bwd(const float *GY, int64_t ldg, const float *X, int64_t ldx, const uint8_t *mask,
                               const float *stats, const float *gamma, const float *beta, int64_t rows, int32_t F,
                               float p_drop, float *GX, int64_t ldgx, float *partial, size_t partial_bytes,
                               float *dgamma, float *dbeta, void *stream);

/* y = relu(x) * keep / (1 - p), one pass, Y may alias X (the GCN layers' relu followed by dropout); the same
 * counter-based keep-bits as above.  mask: rows * F/4 bytes, bit i of a chunk set = element i positive and
 * kept; backward is gx = gy * mask / (1 - p) (GX may alias GY).  F % 4 == 0, rows 16-byte aligned. */
int gnnagg_relu_dropout_fwd(const float *X, int64_t ldx, int64_t rows, int32_t F, float p_drop, uint64_t seed,
                            float *Y, int64_t ldy, uint8_t *mask, void *stream);
int gnnagg_relu_dropout_bwd(const float *GY, int64_t ldg, const uint8_t *mask, int64_t rows, int32_t F, float p_drop,
                            float *GX, int64_t ldgx, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* GNNAGG_H */
