"""Aggregator forward / backward on the "push" transport (Communicator(transport="push")).

Same arithmetic as the all-to-all path of aggregator.py; what changes is how halo rows travel:
the kernel `gnnagg_push_rows` stores them straight into the receivers' buffers (peer memory), on a
side stream, and a 4-byte all-reduce queued behind the stores tells every rank that its rows are in.

  forward   [free?] push(x[idx] | packed codes+params | pre-aggregated rows) -> signal        (side stream)
            (push = the store kernel, or with Communicator(push_engine="copy") one device-to-device copy per
            peer on the copy engines, after a gather into the send buffer where the rows are not contiguous)
            local SpMM                                                                        (compute)
            wait signal -> remote / post SpMM -> raise "free" for the next forward            (compute)
  backward  transposed receive-side SpMM (packs in its epilogue when the halo is packed) ->
            push -> signal; local transposed SpMM; wait -> scatter-add / transposed pre-aggregation

With the fp32 halo on the plain path the peers are served in `Communicator.push_groups` groups
(group g = the peers rank+1+g*k ... ), each with its own signal, and the receive-side SpMM runs
group by group on per-peer slices of remote_adj_t while later groups are still in flight.  Rows of
one destination are then added in arrival order instead of ascending peer order (same terms, fp32
re-association); one group reproduces the all-to-all path bit for bit.

A buffer is only overwritten by a peer after that peer has seen a signal every rank raised behind its
last use of the buffer: the "free" signal for the consumer side, the next "rows are in" signal for
the producer side (the role swap of the reference's buffers in backward).
"""
import torch

from .communicator import Communicator
from .quantizer import Quantizer_for_all_procs
from .spmm_kernel import (SPMM_backward, SPMM_backward_packed, SPMM_backward_quant_pack, SPMM_forward,
                          SPMM_forward_packed, SPMM_forward_quant_pack, quant_pack_fusable)


def _groups(P: int, rank: int, n_groups: int):
    """[(first_peer, num_peers, [source ranks whose rows arrive with this group])]: group g serves the
    peers rank+1+g*k ..., and by symmetry receives from rank-1-g*k ... ."""
    n_groups = max(1, min(n_groups, P - 1))
    k = -(-(P - 1) // n_groups)
    out = []
    for s0 in range(1, P, k):
        cnt = min(k, P - s0)
        out.append(((rank + s0) % P, cnt, [(rank - s) % P for s in range(s0, s0 + cnt)]))
    return out


def _bits():
    return Quantizer_for_all_procs.ctx._bits()


def _side_stream(cur):
    """The stream the stores run on, ordered behind the work already queued on `cur`."""
    side = Communicator.ctx.push_stream(cur.device)
    side.wait_stream(cur)
    return side


def _push(plan, direction, cur, jobs, groups):
    """jobs = [(payload, src tensor, row_bytes, idx)] stored group by group on the side stream; returns one
    signal per group."""
    side = _side_stream(cur)
    signals = []
    with torch.cuda.stream(side):
        if plan.free[direction] is not None:
            plan.free[direction].wait()  # every receiver is done with what the last exchange left there
            plan.free[direction] = None
        for first, cnt, _ in groups:
            for payload, src, row_bytes, idx in jobs:
                plan.push(direction, payload, src, row_bytes, first, cnt, idx)
            signals.append(plan.peers.signal())
    for _, src, _, idx in jobs:  # the side stream still reads them after the caller moves on
        src.record_stream(side)
        if idx is not None:
            idx.record_stream(side)
    return signals


def forward(graph, x, feat_len, num_bits, is_pre_delay, packed, world_size, rec):
    from .aggregator import (_fuse_pack as fuse_pack, _fuse_unpack_forward as fuse_unpack_forward, _prefix as prefix,
                             _remote_parts as remote_parts, _resize as resize, _send_idx as send_idx, gather_rows)

    plan = graph.push_plan
    P, r = world_size, plan.rank
    cur = torch.cuda.current_stream(x.device)
    t = rec.start() if rec else None
    resize(graph, feat_len, num_bits)
    q = graph.comm_buf_for_quantization
    n_groups = Communicator.ctx.push_groups if (not packed and not is_pre_delay) else 1
    groups = _groups(P, r, n_groups)
    if packed:
        if is_pre_delay and fuse_pack(graph) and quant_pack_fusable(x):
            SPMM_forward_quant_pack(graph.adj_t_pre_post_aggr_to, x, q.quantized_send_data_buf,
                                    q.quantized_send_params_buf_fp32, q.quantized_send_params_buf_bf16,
                                    q.quantized_work_range_per_proc, P, _bits())
        elif is_pre_delay:
            if getattr(graph.comm_buf, "lean", False):
                raise RuntimeError("lean halo buffers: feature rows must suit the fused pack kernel")
            SPMM_forward(graph.adj_t_pre_post_aggr_to, x, graph.comm_buf.send_buf, accumulate=False)
            Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(
                graph.comm_buf.send_buf, q.quantized_send_data_buf, q.quantized_send_params_buf_fp32,
                q.quantized_work_range_per_proc, params_bf16=q.quantized_send_params_buf_bf16)
        else:
            Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(
                x, q.quantized_send_data_buf, q.quantized_send_params_buf_fp32, q.quantized_work_range_per_proc,
                params_bf16=q.quantized_send_params_buf_bf16, gather_idx=send_idx(graph))
        jobs = [("codes", q.quantized_send_data_buf, feat_len, None), ("params", q.quantized_send_params_buf_bf16, 4, None)]
    elif is_pre_delay:
        SPMM_forward(graph.adj_t_pre_post_aggr_to, x, graph.comm_buf.send_buf, accumulate=False)
        jobs = [("rows", graph.comm_buf.send_buf, 4 * feat_len, None)]
    elif plan.peers.engine == "copy":
        # copy engines move contiguous blocks: gather the rows into the send buffer first (after the last
        # backward's rows, which peers stored there, have been consumed: stream order on this rank)
        gather_rows(x, send_idx(graph), graph.comm_buf.send_buf)
        jobs = [("rows", graph.comm_buf.send_buf, 4 * feat_len, None)]
    else:
        jobs = [("rows", x, 4 * feat_len, send_idx(graph))]  # the gather is part of the store kernel
    signals = _push(plan, "forward", cur, jobs, groups)
    if rec:
        rec.record_prepare_comm_time(t)

    t = rec.start() if rec else None
    out = torch.empty([graph.local_adj_t.sparse_size(0), feat_len], dtype=torch.float32, device=x.device)
    SPMM_forward(graph.local_adj_t, x, out, accumulate=False)
    if rec:
        rec.record_local_aggregate_time(t)

    t = rec.start() if rec else None
    adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t
    have_rows = sum(graph.comm_splits.recv_splits) != 0
    if len(groups) == 1:
        signals[0].wait()
        if have_rows:
            if packed and fuse_unpack_forward(graph, feat_len):
                SPMM_forward_packed(adj, q.quantized_recv_data_buf, q.quantized_recv_params_buf_bf16,
                                    q.dequantized_work_range_per_proc, P, _bits(), out)
            elif packed:  # narrow rows: unpack into the fp32 halo buffer, then the plain SpMM
                Quantizer_for_all_procs.ctx.dequantize_intX_to_fp32(
                    q.quantized_recv_data_buf, graph.comm_buf.recv_buf, q.quantized_recv_params_buf_fp32,
                    q.dequantized_work_range_per_proc, params_bf16=q.quantized_recv_params_buf_bf16)
                SPMM_forward(adj, graph.comm_buf.recv_buf, out)
            else:
                SPMM_forward(adj, graph.comm_buf.recv_buf, out)
    else:
        parts = remote_parts(graph, P)
        offs = prefix(graph.comm_splits.recv_splits)
        for (_, _, sources), sig in zip(groups, signals):
            sig.wait()
            for src in sources:
                if parts[src] is not None:
                    SPMM_forward(parts[src], graph.comm_buf.recv_buf[offs[src]:offs[src + 1]], out)
    plan.free["forward"] = plan.peers.signal()  # behind the SpMMs above: this rank is done reading
    if rec:
        rec.record_remote_aggregate_time(t)
    return out


def backward(graph, g, feat_len, num_bits, is_pre_delay, packed, world_size, rec):
    from .aggregator import (_fuse_pack as fuse_pack, _prefix as prefix, _remote_parts as remote_parts,
                             _resize as resize, _scatter_adj as scatter_adj)

    plan = graph.push_plan
    P, r = world_size, plan.rank
    cur = torch.cuda.current_stream(g.device)
    resize(graph, feat_len, num_bits)
    q = graph.comm_buf_for_quantization
    adj = graph.adj_t_pre_post_aggr_from if is_pre_delay else graph.remote_adj_t
    have_halo = sum(graph.comm_splits.recv_splits) != 0
    n_groups = Communicator.ctx.push_groups if (not packed and not is_pre_delay) else 1
    groups = _groups(P, r, n_groups)
    t = rec.start() if rec else None
    if packed:
        if have_halo and fuse_pack(graph) and quant_pack_fusable(g):
            SPMM_backward_quant_pack(adj, g, q.quantized_recv_data_buf, q.quantized_recv_params_buf_fp32,
                                     q.quantized_recv_params_buf_bf16, q.dequantized_work_range_per_proc, P, _bits())
        elif have_halo:
            if getattr(graph.comm_buf, "lean", False):
                raise RuntimeError("lean halo buffers: gradient rows must suit the fused pack kernel")
            SPMM_backward(adj, g, graph.comm_buf.recv_buf, accumulate=False)
            Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(
                graph.comm_buf.recv_buf, q.quantized_recv_data_buf, q.quantized_recv_params_buf_fp32,
                q.dequantized_work_range_per_proc, params_bf16=q.quantized_recv_params_buf_bf16)
        signals = _push(plan, "backward", cur, [("codes", q.quantized_recv_data_buf, feat_len, None),
                                                ("params", q.quantized_recv_params_buf_bf16, 4, None)], groups)
    elif len(groups) == 1:
        if have_halo:
            SPMM_backward(adj, g, graph.comm_buf.recv_buf, accumulate=False)
        signals = _push(plan, "backward", cur, [("rows", graph.comm_buf.recv_buf, 4 * feat_len, None)], groups)
    else:
        # the block that goes back to a group of peers is produced right before that group is served
        parts = remote_parts(graph, P)
        offs = prefix(graph.comm_splits.recv_splits)
        signals = []
        for first, cnt, _ in groups:
            for j in range(cnt):
                dst = (first + j) % P
                if parts[dst] is not None:
                    SPMM_backward(parts[dst], g, graph.comm_buf.recv_buf[offs[dst]:offs[dst + 1]], accumulate=False)
            signals += _push(plan, "backward", cur, [("rows", graph.comm_buf.recv_buf, 4 * feat_len, None)],
                             [(first, cnt, None)])
    if rec:
        rec.record_pre_aggregate_time(t)

    t = rec.start() if rec else None
    grad = torch.empty([graph.local_adj_t.sparse_size(-1), feat_len], dtype=torch.float32, device=g.device)
    SPMM_backward(graph.local_adj_t, g, grad, accumulate=False)
    if rec:
        rec.record_local_aggregate_time(t)

    t = rec.start() if rec else None
    for sig in signals:
        sig.wait()
    if sum(graph.comm_splits.send_splits) != 0:
        if packed:
            args = (q.quantized_send_data_buf, q.quantized_send_params_buf_bf16, q.quantized_work_range_per_proc, P,
                    _bits(), grad)
            if is_pre_delay:
                SPMM_backward_packed(graph.adj_t_pre_post_aggr_to, *args)
            else:
                SPMM_forward_packed(scatter_adj(graph), *args)
        elif is_pre_delay:
            SPMM_backward(graph.adj_t_pre_post_aggr_to, graph.comm_buf.send_buf, grad)
        else:
            SPMM_forward(scatter_adj(graph), graph.comm_buf.send_buf, grad)
    plan.free["backward"] = plan.peers.signal()
    if rec:
        rec.record_remote_aggregate_time(t)
    return grad
