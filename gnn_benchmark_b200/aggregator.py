"""Aggregator: the autograd aggregation op of the GNN layers, on CUDA kernels.

Same call as the reference (self_benchmark/a64fx/model/layers/aggregator.py:15-208):
    out = Aggregator.apply(graph, local_nodes_feat, layer, num_bits, is_pre_delay, is_training)

forward  out = A_local @ x  +  A_remote @ halo(x)          (aggregator.py:17-119)
backward grad = A_local^T @ g + scatter(halo^T(A_remote^T @ g))   (aggregator.py:121-208)

Per call, on the current (compute) stream unless noted:
  1. fill the send side: pre-aggregation SpMM (pre/post path) or row gather; with a packed halo the
     quantise + pack step is the epilogue of that SpMM / fused with that gather, so no fp32 send
     buffer is written (backward: the transposed receive-side SpMM packs its rows the same way);
  2. start the exchange (Communicator; runs on the NCCL stream);
  3. local SpMM, overlapping the exchange;
  4. make the compute stream wait for the exchange, unpack + dequantise if it was packed;
  5. remote / post-aggregation SpMM accumulating onto the local result (forward), or
     the transposed pre-aggregation SpMM / deterministic scatter-add (backward).
The output tensors are written by the first SpMM (accumulate off), so no zero fill is needed.
"""
import torch
import torch.distributed as dist

from . import _lib
from .communicator import Communicator
from .quantizer import Quantizer_for_all_procs
from .spmm_kernel import (SPMM_backward, SPMM_backward_packed, SPMM_backward_quant_pack, SPMM_forward,
                          SPMM_forward_packed, SPMM_forward_quant_pack, quant_pack_fusable)
from .time_recorder import TimeRecorder


# Packed halo modes: decode the received codes inside the receive-side SpMM instead of unpacking them
# into the fp32 halo buffer first (same result bit for bit; the fp32 buffer is then left untouched).
# Set to False to get the reference's two-step sequence, e.g. to inspect comm_buf.recv_buf.
FUSE_UNPACK = True
# ... in forward only from this width on: below it the unpack kernel followed by the fp32 SpMM is the faster
# pair (1.9 M halo rows, 65 M nonzeros, 2 bits: 2.11 vs 2.58 ms at 32 columns, 3.57 vs 3.81 at 128, 7.50 vs 6.88
# at 256; the packed SpMM pays a slot -> (row, shift, parameters) lookup per nonzero, which wide rows amortise).
# The backward scatter is fused at every width (fused is never slower there), and so is everything when the
# fp32 halo buffers do not exist (lean halo buffers).
FUSE_UNPACK_MIN_WIDTH = 192
# Packed halo modes: quantise + pack as the epilogue of the SpMM that produces the rows to send (forward:
# pre-aggregation; backward: transposed receive-side matrix), so comm_buf.send_buf / recv_buf are never
# written.  "lean": only where those fp32 buffers do not exist (lean halo buffers) -- with the buffers there,
# SpMM into them followed by the pack kernel is the faster pair below 256 columns (the encoder inside the
# SpMM costs instruction-cache misses); True: always; False: never (the reference's two-step sequence).
FUSE_PACK = "lean"


def _fuse_unpack_forward(graph, feat_len: int) -> bool:
    if not FUSE_UNPACK or feat_len % 4 != 0:
        return False
    return feat_len >= FUSE_UNPACK_MIN_WIDTH or bool(getattr(graph.comm_buf, "lean", False))


def _fuse_pack(graph) -> bool:
    if FUSE_PACK == "lean":
        return bool(getattr(graph.comm_buf, "lean", False))
    return bool(FUSE_PACK)


def _world_size() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def gather_rows(x: torch.Tensor, idx_i32: torch.Tensor, out: torch.Tensor) -> None:
    """out[i, :] = x[idx[i], :] (replaces torch.index_select(..., out=send_buf), aggregator.py:51)."""
    _lib.require_cuda(x, idx_i32, out)
    rows, F = idx_i32.numel(), x.size(1)
    if rows == 0:
        return
    rc = _lib.lib().gnnagg_gather_rows_f32(x.data_ptr(), x.stride(0), idx_i32.data_ptr(), rows, F, out.data_ptr(),
                                           out.stride(0), _lib.stream_ptr(x.device))
    _lib.check(rc, "gather_rows_f32")


def _packed(num_bits: int, graph) -> bool:
    comm = Communicator.ctx
    bits = comm.num_bits if comm is not None else num_bits
    return bits in (2, 4, 8) and graph.comm_buf_for_quantization is not None


def _resize(graph, feat_len: int, num_bits: int) -> None:
    graph.comm_buf.resize_buffer(graph.comm_splits, feat_len, num_bits)
    if num_bits != 32 and num_bits != 16 and graph.comm_buf_for_quantization is not None:
        graph.comm_buf_for_quantization.resize_buffer(graph.comm_splits, feat_len, num_bits)


def _rec():
    return TimeRecorder.ctx


def _prefix(splits):
    out = [0]
    for x in splits:
        out.append(out[-1] + x)
    return out


def _remote_parts(graph, world_size):
    """remote_adj_t cut into one matrix per source peer (columns = that peer's halo slots, renumbered
    from 0), built on first use and cached on the graph.  Rows keep CSR order, so applying the parts
    one after the other in ascending peer order is the same FMA chain as the whole matrix."""
    parts = getattr(graph, "_remote_parts", None)
    if parts is None:
        from .sparse import SparseTensor
        rowptr, col, val = graph.remote_adj_t.csr()
        n = graph.remote_adj_t.sparse_size(0)
        rows = torch.repeat_interleave(torch.arange(n, device=col.device), rowptr[1:] - rowptr[:-1])
        offs = _prefix(graph.comm_splits.recv_splits)
        parts = []
        for p in range(world_size):
            lo, hi = offs[p], offs[p + 1]
            if hi == lo:
                parts.append(None)
                continue
            m = (col >= lo) & (col < hi)
            parts.append(SparseTensor(row=rows[m], col=col[m].to(torch.int64) - lo, value=val[m],
                                      sparse_sizes=(n, hi - lo), is_sorted=True))
        graph._remote_parts = parts
    return parts


def _push_transport(graph) -> bool:
    comm = Communicator.ctx
    return comm is not None and comm.transport == "push" and getattr(graph, "push_plan", None) is not None


def _pipelined(num_bits, is_pre_delay, is_training, world_size) -> bool:
    comm = Communicator.ctx
    fp32 = comm is not None and (comm.num_bits == 32 or not is_training)
    return world_size > 1 and fp32 and not is_pre_delay and comm.pipeline_peers


class Aggregator(torch.autograd.Function):
    @staticmethod
    def forward(ctx, graph, local_nodes_feat, layer, num_bits: int, is_pre_delay: bool, is_training: bool):
        ctx.graph = graph
        ctx.num_bits = num_bits
        ctx.is_pre_delay = is_pre_delay
        ctx.layer = layer

        world_size = _world_size()
        rec = _rec()
        t_total = rec.start() if rec else None
        # rows may be padded (row stride > F, e.g. 100-wide features kept in 128-float rows so that every
        # gathered row starts on a 128-byte line); every kernel on the path takes a leading dimension
        x = local_nodes_feat
        if x.dim() != 2 or x.stride(1) != 1 or x.stride(0) < x.size(1):
            x = x.contiguous()
        feat_len = x.size(-1)
        lean = bool(getattr(graph.comm_buf, "lean", False))  # no fp32 staging buffers: the halo stays packed
        packed = world_size > 1 and (is_training or lean) and _packed(num_bits, graph)

        comm_handle = None
        rounds = None
        if world_size > 1 and _push_transport(graph):
            from . import aggregator_push

            out = aggregator_push.forward(graph, x, feat_len, num_bits, is_pre_delay, packed, world_size, rec)
            if rec:
                rec.record_total_convolution_time(t_total)
                rec.next_layer()
            return out
        if _pipelined(num_bits, is_pre_delay, is_training, world_size):
            # peer-by-peer exchange: every peer's rows are aggregated as soon as they are in
            t = rec.start() if rec else None
            _resize(graph, feat_len, num_bits)
            gather_rows(x, _send_idx(graph), graph.comm_buf.send_buf)
            if rec:
                rec.record_prepare_comm_time(t)
            rounds = Communicator.ctx.exchange_by_peer(graph.comm_buf.send_buf, graph.comm_buf.recv_buf,
                                                       graph.comm_splits.send_splits, graph.comm_splits.recv_splits)
        elif world_size > 1:
            t = rec.start() if rec else None
            _resize(graph, feat_len, num_bits)
            send_buf = graph.comm_buf.send_buf
            q = graph.comm_buf_for_quantization
            fused_pack = False
            if is_pre_delay and packed and _fuse_pack(graph) and quant_pack_fusable(x):
                # pre-aggregation with the quantise + pack step as its epilogue
                SPMM_forward_quant_pack(graph.adj_t_pre_post_aggr_to, x, q.quantized_send_data_buf,
                                        q.quantized_send_params_buf_fp32, q.quantized_send_params_buf_bf16,
                                        q.quantized_work_range_per_proc, world_size, Quantizer_for_all_procs.ctx._bits())
                fused_pack = True
            elif is_pre_delay:  # pre-aggregation: partial sums for remote destinations, raw rows for post sources
                SPMM_forward(graph.adj_t_pre_post_aggr_to, x, send_buf, accumulate=False)
            elif packed:      # gather fused into quantise + pack
                Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(
                    x, q.quantized_send_data_buf, q.quantized_send_params_buf_fp32, q.quantized_work_range_per_proc,
                    params_bf16=q.quantized_send_params_buf_bf16, gather_idx=_send_idx(graph))
                fused_pack = True
            else:
                gather_rows(x, _send_idx(graph), send_buf)
            if rec:
                rec.record_prepare_comm_time(t)
            if lean and not fused_pack:
                raise RuntimeError("lean halo buffers need a packed halo and feature rows the fused pack kernels take "
                                   "(F a multiple of 4, at most 512, 16-byte aligned rows)")
            if fused_pack:
                comm_handle = Communicator.ctx.comm_with_int2_quantization_for_all_procs(
                    graph.comm_splits, graph.comm_buf, q, "forward", already_quantized=True)
            else:
                comm_handle = Communicator.ctx.comm(graph.comm_splits, graph.comm_buf, q, f"forward{layer}",
                                                    is_training, "forward")

        t = rec.start() if rec else None
        out = torch.empty([graph.local_adj_t.sparse_size(0), feat_len], dtype=torch.float32, device=x.device)
        SPMM_forward(graph.local_adj_t, x, out, accumulate=False)
        if rec:
            rec.record_local_aggregate_time(t)

        if comm_handle is not None:
            comm_handle.wait()

        if rounds is not None:
            t = rec.start() if rec else None
            parts = _remote_parts(graph, world_size)
            offs = _prefix(graph.comm_splits.recv_splits)
            for src, works in rounds:
                for w in works:
                    w.wait()
                if parts[src] is not None:
                    SPMM_forward(parts[src], graph.comm_buf.recv_buf[offs[src]:offs[src + 1]], out)
            if rec:
                rec.record_remote_aggregate_time(t)
                rec.record_total_convolution_time(t_total)
                rec.next_layer()
            return out

        num_recv_nodes = sum(graph.comm_splits.recv_splits) if world_size > 1 else 0
        fused = packed and _fuse_unpack_forward(graph, feat_len)
        if packed and num_recv_nodes != 0 and not fused:
            t = rec.start() if rec else None
            q = graph.comm_buf_for_quantization
            Quantizer_for_all_procs.ctx.dequantize_intX_to_fp32(
                q.quantized_recv_data_buf, graph.comm_buf.recv_buf, q.quantized_recv_params_buf_fp32,
                q.dequantized_work_range_per_proc, params_bf16=q.quantized_recv_params_buf_bf16)
            if rec:
                rec.record_dequantization_time(t)

        if world_size > 1 and num_recv_nodes != 0:
            t = rec.start() if rec else None
            adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t  # post-aggregation / remote
            if fused:
                q = graph.comm_buf_for_quantization
                SPMM_forward_packed(adj, q.quantized_recv_data_buf, q.quantized_recv_params_buf_bf16,
                                    q.dequantized_work_range_per_proc, world_size, Quantizer_for_all_procs.ctx._bits(),
                                    out)
            else:
                SPMM_forward(adj, graph.comm_buf.recv_buf, out)
            if rec:
                rec.record_remote_aggregate_time(t)

        if rec:
            rec.record_total_convolution_time(t_total)
            rec.next_layer()
        return out

    @staticmethod
    def backward(ctx, local_out_grad):
        graph = ctx.graph
        num_bits = ctx.num_bits
        is_pre_delay = ctx.is_pre_delay
        layer = f"backward{ctx.layer}"

        world_size = _world_size()
        rec = _rec()
        t_total = rec.start() if rec else None
        g = local_out_grad.contiguous()
        feat_len = g.size(-1)
        packed = world_size > 1 and _packed(num_bits, graph)

        comm_handle = None
        rounds = None
        if world_size > 1 and _push_transport(graph):
            from . import aggregator_push

            grad = aggregator_push.backward(graph, g, feat_len, num_bits, is_pre_delay, packed, world_size, rec)
            if rec:
                rec.record_total_convolution_time(t_total)
                rec.next_layer()
            return None, grad, None, None, None, None
        if _pipelined(num_bits, is_pre_delay, True, world_size):
            # the block of halo gradients that goes back to a peer is computed right before its round
            _resize(graph, feat_len, num_bits)
            parts = _remote_parts(graph, world_size)
            offs = _prefix(graph.comm_splits.recv_splits)
            t = rec.start() if rec else None

            def make_block(dst):
                if parts[dst] is not None:
                    SPMM_backward(parts[dst], g, graph.comm_buf.recv_buf[offs[dst]:offs[dst + 1]], accumulate=False)

            rounds = Communicator.ctx.exchange_by_peer(graph.comm_buf.recv_buf, graph.comm_buf.send_buf,
                                                       graph.comm_splits.recv_splits, graph.comm_splits.send_splits,
                                                       before_send=make_block)
            if rec:
                rec.record_pre_aggregate_time(t)
        elif world_size > 1 and packed and _fuse_pack(graph) and quant_pack_fusable(g):
            # halo gradients: the transposed receive-side SpMM packs its rows in its epilogue, so the fp32
            # halo buffer is never needed (the receive-side buffers are the ones sent: the roles swap)
            _resize(graph, feat_len, num_bits)
            t = rec.start() if rec else None
            q = graph.comm_buf_for_quantization
            adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t
            if sum(graph.comm_splits.recv_splits) != 0:
                SPMM_backward_quant_pack(adj, g, q.quantized_recv_data_buf, q.quantized_recv_params_buf_fp32,
                                         q.quantized_recv_params_buf_bf16, q.dequantized_work_range_per_proc,
                                         world_size, Quantizer_for_all_procs.ctx._bits())
            if rec:
                rec.record_pre_aggregate_time(t)
            comm_handle = Communicator.ctx.comm_with_int2_quantization_for_all_procs(
                graph.comm_splits, graph.comm_buf, graph.comm_buf_for_quantization, "backward",
                already_quantized=True)
        elif world_size > 1:
            if getattr(graph.comm_buf, "lean", False):
                raise RuntimeError("lean halo buffers need a packed halo and gradient rows the fused pack kernel takes "
                                   "(F a multiple of 4, at most 512, 16-byte aligned rows)")
            _resize(graph, feat_len, num_bits)
            # the two buffers swap roles: recv_buf is sent, send_buf receives
            remote_nodes_grad_buf = graph.comm_buf.recv_buf
            t = rec.start() if rec else None
            if remote_nodes_grad_buf.size(0) != 0:
                if is_pre_delay:
                    SPMM_backward(graph.adj_t_pre_post_aggr_from, g, remote_nodes_grad_buf, accumulate=False)
                else:
                    SPMM_backward(graph.remote_adj_t, g, remote_nodes_grad_buf, accumulate=False)
            if rec:
                rec.record_pre_aggregate_time(t)
            comm_handle = Communicator.ctx.comm(graph.comm_splits, graph.comm_buf, graph.comm_buf_for_quantization,
                                                layer, True, "backward")

        t = rec.start() if rec else None
        local_nodes_grad = torch.empty([graph.local_adj_t.sparse_size(-1), feat_len], dtype=torch.float32,
                                       device=g.device)
        SPMM_backward(graph.local_adj_t, g, local_nodes_grad, accumulate=False)
        if rec:
            rec.record_local_aggregate_time(t)

        if comm_handle is not None:
            comm_handle.wait()
        if rounds is not None:
            for _, works in rounds:
                for w in works:
                    w.wait()

        num_recv_nodes = sum(graph.comm_splits.send_splits) if world_size > 1 else 0
        fused = packed and FUSE_UNPACK and feat_len % 4 == 0
        if packed and num_recv_nodes != 0 and not fused:
            t = rec.start() if rec else None
            q = graph.comm_buf_for_quantization
            Quantizer_for_all_procs.ctx.dequantize_intX_to_fp32(
                q.quantized_send_data_buf, graph.comm_buf.send_buf, q.quantized_send_params_buf_fp32,
                q.quantized_work_range_per_proc, params_bf16=q.quantized_send_params_buf_bf16)
            if rec:
                rec.record_dequantization_time(t)

        if world_size > 1 and num_recv_nodes != 0:
            t = rec.start() if rec else None
            local_nodes_grad_buf = graph.comm_buf.send_buf
            if fused:
                q = graph.comm_buf_for_quantization
                args = (q.quantized_send_data_buf, q.quantized_send_params_buf_bf16, q.quantized_work_range_per_proc,
                        world_size, Quantizer_for_all_procs.ctx._bits(), local_nodes_grad)
                if is_pre_delay:
                    SPMM_backward_packed(graph.adj_t_pre_post_aggr_to, *args)
                else:
                    SPMM_forward_packed(_scatter_adj(graph), *args)
            elif is_pre_delay:
                SPMM_backward(graph.adj_t_pre_post_aggr_to, local_nodes_grad_buf, local_nodes_grad)
            else:
                # grad.index_add_(0, idx_nodes_send_to_others, buf) as an accumulating SpMM with the
                # unit scatter matrix: same additions, fixed order, no atomics
                SPMM_forward(_scatter_adj(graph), local_nodes_grad_buf, local_nodes_grad)
            if rec:
                rec.record_remote_aggregate_time(t)

        if rec:
            rec.record_total_convolution_time(t_total)
            rec.next_layer()
        return None, local_nodes_grad, None, None, None, None


def _send_idx(graph) -> torch.Tensor:
    if getattr(graph, "idx_nodes_send_to_others_i32", None) is None:
        graph.idx_nodes_send_to_others_i32 = graph.idx_nodes_send_to_others.to(torch.int32)
    return graph.idx_nodes_send_to_others_i32


def _scatter_adj(graph):
    if getattr(graph, "scatter_adj_t", None) is None:
        from .data_manager.DataLoader import _scatter_matrix
        graph.scatter_adj_t = _scatter_matrix(graph.idx_nodes_send_to_others, graph.local_adj_t.sparse_size(0))
    return graph.scatter_adj_t
