"""Communicator: the halo exchange, with the reference's class and method names
(self_benchmark/a64fx/communicator.py:19-325).

The reference runs MPI / oneCCL all-to-alls between CPU ranks.  Here every rank drives one GPU
and the exchanges are `torch.distributed` all_to_all_single calls on the NCCL backend (grouped
ncclSend/ncclRecv over NVLink): with async_op=True they run on the process group's own stream,
ordered after the work already queued on the caller's stream, and `handle.wait()` makes the
caller's stream (not the host) wait for them -- which is how the exchange overlaps the local
SpMM launched in between.  The blocking barrier the reference puts before every exchange
(communicator.py:98,292) is not needed for correctness and is off by default.

With CPU tensors and the gloo backend the fp32 exchange runs as host-side plumbing (used by the
world_size-2 CPU tests); the bf16 and quantised modes need the CUDA kernels and therefore CUDA
tensors.
"""
import os

import torch
import torch.distributed as dist

from .data_manager import CommBuffer, CommBufferForQuantization, CommSplits
from .quantizer import Quantizer_for_all_procs
from .time_recorder import TimeRecorder
from . import _lib


class _Handles(object):
    """Several async works behind one .wait()."""

    def __init__(self, works):
        self.works = [w for w in works if w is not None]

    def wait(self):
        for w in self.works:
            w.wait()


class Communicator(object):
    ctx = None

    def __init__(self, num_bits=32, is_async=True, use_barrier=False, pipeline_peers=False, transport="all_to_all",
                 push_groups=7, push_engine="auto") -> None:
        """transport (an addition): "all_to_all" -- the reference's exchange, one collective per aggregation
        (NCCL here); "push" -- rows are stored straight into the receivers' buffers over NVLink by the
        kernel that gathers / produces them (peer.py, aggregator_push.py; one node, NCCL process group).
        push_groups: with the fp32 halo on the plain path the peers are served in this many groups (at most one
        per peer), the receive-side SpMM of one group overlapping the stores of the next; 1 keeps the
        ascending-peer summation order of the all-to-all path.  The default is one group per peer on an 8-GPU
        node: measured per step of the aggregation benchmark on 8 GPUs, 1 / 2 / 3 / 4 / 7 groups take
        98.8 / 89.8 / 83.1 / 79.6 / 79.0 ms.
        push_engine: "kernel" -- the store kernel moves the rows (gather fused in, a few SMs busy for the
        length of the exchange); "copy" -- rows are gathered into the send buffer when they are not already
        contiguous and every peer's block travels as one device-to-device copy on the copy engines (no SM);
        "auto" (default) -- copies for blocks that are contiguous as they are (backward, packed halo, pre/post),
        the store kernel where the rows must be gathered (forward, plain plan, fp32).  Measured per step of the
        aggregation benchmark: kernel / copy / auto 53.4 / 54.5 / 54.0 ms on 2 GPUs, 63.4 / 64.8 / 63.6 on 4,
        88.8 / 83.0 / 82.7 on 8."""
        if transport not in ("all_to_all", "push"):
            raise ValueError("transport must be 'all_to_all' or 'push'")
        if push_engine not in ("kernel", "copy", "auto"):
            raise ValueError("push_engine must be 'kernel', 'copy' or 'auto'")
        self.push_engine = push_engine
        self.num_bits = num_bits
        self.is_async = is_async
        self.use_barrier = use_barrier
        self.transport = transport
        self.push_groups = int(push_groups)
        self._peers = None
        self._push_streams = {}
        # fp32 halo only: exchange peer by peer and aggregate each peer's rows as they arrive (see
        # exchange_by_peer).  Off by default because the peers' contributions are then added in arrival
        # order, not in the reference's ascending-peer order (same terms, fp32 re-association).
        self.pipeline_peers = pipeline_peers
        self.world_size = -1
        self.rank = -1
        Communicator.ctx = self

    def init_dist_group(self, backend=None):
        """One process per GPU, launched by torchrun (RANK / WORLD_SIZE / LOCAL_RANK / MASTER_* in
        the environment).  NCCL when CUDA is available, else gloo (communicator.py:28-53 picks
        MPI or oneCCL instead)."""
        if not dist.is_initialized():
            if backend is None:
                backend = "nccl" if torch.cuda.is_available() else "gloo"
            if backend == "nccl":
                local_rank = int(os.environ.get("LOCAL_RANK", 0))
                torch.cuda.set_device(local_rank)
                # the exchange runs on a high-priority stream: its few large CTAs must get onto the SMs
                # while the local SpMM's many small CTAs keep arriving, or the overlap is lost
                opts = dist.ProcessGroupNCCL.Options(is_high_priority_stream=True)
                dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local_rank), pg_options=opts)
            else:
                dist.init_process_group(backend=backend)
        self.world_size = dist.get_world_size()
        self.rank = dist.get_rank()
        return (self.rank, self.world_size)

    def peers(self):
        """The peer-memory service of the push transport (created on first use; tests install their own)."""
        if self._peers is None:
            from .peer import NcclPeers

            self._peers = NcclPeers(torch.device("cuda", torch.cuda.current_device()), engine=self.push_engine)
        return self._peers

    def push_stream(self, device):
        """Side stream of the push transport's stores (high priority: they must get onto the SMs while the
        local SpMM keeps them busy); one per device and host thread."""
        import threading

        key = (torch.device(device).index, threading.get_ident())
        s = self._push_streams.get(key)
        if s is None:
            s = torch.cuda.Stream(device=device, priority=-1)
            self._push_streams[key] = s
        return s

    # ---------------------------------------------------------------------------------------
    def comm(self, comm_splits, comm_buf, comm_buf_for_quantization, layer, is_training, direction):
        """Dispatch on the bit width (communicator.py:55-83): fp32 when num_bits == 32 or outside
        training, bf16 for 16, packed codes for 2 (and here 4 and 8).  Returns an object with
        .wait() or None."""
        comm_handle = None
        lean = bool(getattr(comm_buf, "lean", False))  # no fp32 staging buffers: the halo stays packed in eval too
        if self.num_bits == 32 or (is_training is False and not lean):
            comm_handle = self.comm_with_fp32(comm_splits, comm_buf, direction)
        elif self.num_bits == 16:
            comm_handle = self.comm_with_fp16(comm_splits, comm_buf, direction)
        elif self.num_bits in (2, 4, 8):
            comm_handle = self.comm_with_int2_quantization_for_all_procs(
                comm_splits, comm_buf, comm_buf_for_quantization, direction)
        return comm_handle

    def _barrier(self):
        if self.use_barrier:
            t = TimeRecorder.ctx.start() if TimeRecorder.ctx else None
            dist.barrier()
            if TimeRecorder.ctx:
                TimeRecorder.ctx.record_barrier_time(t)

    def comm_with_fp32(self, comm_splits: CommSplits, comm_buf: CommBuffer, direction: str):
        """communicator.py:85-109."""
        if direction == "forward":
            recv_buf, send_buf = comm_buf.recv_buf, comm_buf.send_buf
            recv_splits, send_splits = comm_splits.recv_splits, comm_splits.send_splits
        else:
            recv_buf, send_buf = comm_buf.send_buf, comm_buf.recv_buf
            recv_splits, send_splits = comm_splits.send_splits, comm_splits.recv_splits
        self._barrier()
        t = TimeRecorder.ctx.start() if TimeRecorder.ctx else None
        handle = dist.all_to_all_single(recv_buf, send_buf, recv_splits, send_splits, async_op=self.is_async)
        if TimeRecorder.ctx:
            TimeRecorder.ctx.record_communication_time(t)
        return handle

    def exchange_by_peer(self, send_buf, recv_buf, send_splits, recv_splits, before_send=None):
        """The fp32 all-to-all as P-1 rounds of one send + one receive (round s: send to rank+s, receive
        from rank-s), each a grouped NCCL send/recv queued on the communication stream.  Returns
        [(source_peer, [work, ...]), ...] in arrival order; waiting on a round's works orders the
        caller's stream after that round only, so the rows of one peer can be aggregated while the
        next peer's rows are still in flight.  `before_send(dst)` (optional) is called right before
        round s is queued, to produce the block that goes to `dst` (backward direction)."""
        P, r = dist.get_world_size(), dist.get_rank()
        so = [0]
        for x in send_splits:
            so.append(so[-1] + x)
        ro = [0]
        for x in recv_splits:
            ro.append(ro[-1] + x)
        rounds = []
        rec = TimeRecorder.ctx
        t = rec.start() if rec else None
        for s in range(1, P):
            dst, src = (r + s) % P, (r - s) % P
            if before_send is not None:
                before_send(dst)
            ops = []
            if send_splits[dst]:
                ops.append(dist.P2POp(dist.isend, send_buf[so[dst]:so[dst + 1]], dst))
            if recv_splits[src]:
                ops.append(dist.P2POp(dist.irecv, recv_buf[ro[src]:ro[src + 1]], src))
            rounds.append((src, dist.batch_isend_irecv(ops) if ops else []))
        if rec:
            rec.record_communication_time(t)
        return rounds

    def comm_with_fp16(self, comm_splits: CommSplits, comm_buf: CommBuffer, direction: str):
        """bf16 on the wire (communicator.py:111-143).  The reference widens the received buffer
        before waiting for the exchange (:137, a race when async); here the widening is queued
        behind the exchange and the returned handle covers both."""
        if direction == "forward":
            recv_buf, send_buf = comm_buf.recv_buf, comm_buf.send_buf
            recv_buf_fp16, send_buf_fp16 = comm_buf.recv_buf_fp16, comm_buf.send_buf_fp16
            recv_splits, send_splits = comm_splits.recv_splits, comm_splits.send_splits
        else:
            recv_buf, send_buf = comm_buf.send_buf, comm_buf.recv_buf
            recv_buf_fp16, send_buf_fp16 = comm_buf.send_buf_fp16, comm_buf.recv_buf_fp16
            recv_splits, send_splits = comm_splits.send_splits, comm_splits.recv_splits
        rec = TimeRecorder.ctx
        t = rec.start() if rec else None
        _cast(send_buf, send_buf_fp16)
        if rec:
            rec.record_quantization_time(t)
        t = rec.start() if rec else None
        handle = dist.all_to_all_single(recv_buf_fp16, send_buf_fp16, recv_splits, send_splits,
                                        async_op=self.is_async)
        if rec:
            rec.record_communication_time(t)
        return _CastAfter(handle, recv_buf_fp16, recv_buf)

    def comm_with_int2_quantization_for_all_procs(self, comm_splits: CommSplits, comm_buf: CommBuffer,
                                                  comm_buf_for_quantization: CommBufferForQuantization,
                                                  direction: str, already_quantized: bool = False):
        """Quantise + pack the send buffer, exchange the bf16 parameters, then the packed codes
        (communicator.py:231-325).  The fp32 -> bf16 cast of the parameters (:297) is done by the
        pack kernel; the bf16 -> fp32 widening (:303) by the unpack kernel on the receive side.
        `already_quantized`: the caller filled the code / parameter buffers itself (fused
        gather + pack)."""
        q = comm_buf_for_quantization
        if direction == "forward":
            recv_splits, send_splits = comm_splits.recv_splits, comm_splits.send_splits
            recv_splits_int2, send_splits_int2 = comm_splits.recv_splits_int2, comm_splits.send_splits_int2
            send_buf = comm_buf.send_buf
            quantized_recv_data_buf, quantized_send_data_buf = q.quantized_recv_data_buf, q.quantized_send_data_buf
            recv_params_bf16, send_params_bf16 = q.quantized_recv_params_buf_bf16, q.quantized_send_params_buf_bf16
            send_params_fp32 = q.quantized_send_params_buf_fp32
            quantized_work_range_per_proc = q.quantized_work_range_per_proc
        else:
            recv_splits, send_splits = comm_splits.send_splits, comm_splits.recv_splits
            recv_splits_int2, send_splits_int2 = comm_splits.send_splits_int2, comm_splits.recv_splits_int2
            send_buf = comm_buf.recv_buf
            quantized_recv_data_buf, quantized_send_data_buf = q.quantized_send_data_buf, q.quantized_recv_data_buf
            recv_params_bf16, send_params_bf16 = q.quantized_send_params_buf_bf16, q.quantized_recv_params_buf_bf16
            send_params_fp32 = q.quantized_recv_params_buf_fp32
            quantized_work_range_per_proc = q.dequantized_work_range_per_proc

        rec = TimeRecorder.ctx
        if not already_quantized:
            t = rec.start() if rec else None
            Quantizer_for_all_procs.ctx.quantize_fp32_to_intX(
                send_buf, quantized_send_data_buf, send_params_fp32, quantized_work_range_per_proc,
                params_bf16=send_params_bf16)
            if rec:
                rec.record_quantization_time(t)
        self._barrier()
        t = rec.start() if rec else None
        handle = self._exchange_together([
            (recv_params_bf16, send_params_bf16, recv_splits, send_splits),
            (quantized_recv_data_buf, quantized_send_data_buf, recv_splits_int2, send_splits_int2)])
        if rec:
            rec.record_communication_time(t)
        return handle

    def comm_with_mixed_quantization(self, recv_buf, send_buf, recv_splits, send_splits, nodes_num_bits_tensor):
        """Halo exchange with a bit width per row (communicator.py:383-489 of the reference; there the
        call from comm() is commented out, the method itself is complete).  Every row of send_buf is
        quantised with its own width from nodes_num_bits_tensor (8 / 4 / 2; fp32, one value per row) into
        a ragged byte buffer (row i at [range[i], range[i+1]), range = cumsum(ceil(bits_i * F / 8))); the
        parameters [bits, zero_point, scale] travel first, as bf16, so that the receiver can size its
        byte buffer; then the codes.  Returns, like the reference,
            (handle of the code exchange, quantized_recv_buf, dequantized_nodes_feat_range, dequantized_params)
        for QuantizerForMixedBits.dequantize_intX_to_fp32(quantized_recv_buf, recv_buf, range, params)
        after handle.wait().  The parameters the receiver decodes with are the bf16-rounded ones."""
        from .quantizer import QuantizerForMixedBits

        rec = TimeRecorder.ctx
        dev = send_buf.device
        num_send_nodes, num_recv_nodes = int(sum(send_splits)), int(sum(recv_splits))
        feat_len = send_buf.size(1)
        t = rec.start() if rec else None
        send_params = torch.empty((num_send_nodes, 3), dtype=torch.float32, device=dev)
        send_params[:, 0] = nodes_num_bits_tensor.to(dev)
        quantized_nodes_feat_range = QuantizerForMixedBits.get_quantized_nodes_feat_range(
            num_send_nodes, feat_len, send_params[:, 0])
        quantized_send_buf = torch.empty(int(quantized_nodes_feat_range[-1].item()), dtype=torch.uint8, device=dev)
        QuantizerForMixedBits.quantize_fp32_to_intX(send_buf, quantized_send_buf, quantized_nodes_feat_range, send_params)
        if rec:
            rec.record_quantization_time(t)
        t = rec.start() if rec else None
        recv_params = torch.empty((num_recv_nodes, 3), dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(recv_params, send_params.to(torch.bfloat16), list(recv_splits), list(send_splits),
                               async_op=False)
        dequantized_params = recv_params.to(torch.float32)
        dequantized_nodes_feat_range = QuantizerForMixedBits.get_quantized_nodes_feat_range(
            num_recv_nodes, feat_len, dequantized_params[:, 0])
        quantized_recv_splits, quantized_send_splits = self.get_splits_for_comm_quantized_data(
            recv_splits, send_splits, dequantized_nodes_feat_range, quantized_nodes_feat_range)
        quantized_recv_buf = torch.empty(int(dequantized_nodes_feat_range[-1].item()), dtype=torch.uint8, device=dev)
        comm_handle = dist.all_to_all_single(quantized_recv_buf, quantized_send_buf, quantized_recv_splits,
                                             quantized_send_splits, async_op=self.is_async)
        if rec:
            rec.record_communication_time(t)
        return comm_handle, quantized_recv_buf, dequantized_nodes_feat_range, dequantized_params

    @staticmethod
    def get_splits_for_comm_quantized_data(recv_splits, send_splits, dequantized_nodes_feat_range,
                                           quantized_nodes_feat_range):
        """Bytes per peer of the ragged code buffers (communicator.py:327-381): differences of the byte
        ranges at the per-peer row boundaries."""
        def per_peer(splits, byte_range):
            rows = torch.zeros(len(splits) + 1, dtype=torch.int64)
            rows[1:] = torch.as_tensor(splits, dtype=torch.int64).cumsum(0)
            at = byte_range.to("cpu")[rows]
            return (at[1:] - at[:-1]).tolist()

        return per_peer(recv_splits, dequantized_nodes_feat_range), per_peer(send_splits, quantized_nodes_feat_range)

    def _exchange_together(self, parts):
        """Several all-to-alls with row splits -- parts = [(recv, send, recv_splits, send_splits), ...] --
        as ONE exchange.  The reference sends the parameters and the codes of a packed halo as two
        messages per peer (communicator.py:297-311).  On NCCL both travel in one grouped launch of
        point-to-point operations (every rank lists its sends and receives per peer in the same part
        order, so they pair up); other backends (the gloo plumbing tests) run one all_to_all_single per
        part."""
        if dist.get_backend() != "nccl":
            return _Handles([dist.all_to_all_single(r, s, rs, ss, async_op=self.is_async) for r, s, rs, ss in parts])
        ops = []
        for recv, send, recv_splits, send_splits in parts:
            ro = so = 0
            for p, (nr, ns) in enumerate(zip(recv_splits, send_splits)):
                if ns:
                    ops.append(dist.P2POp(dist.isend, send[so:so + ns], p))
                if nr:
                    ops.append(dist.P2POp(dist.irecv, recv[ro:ro + nr], p))
                ro, so = ro + nr, so + ns
        works = dist.batch_isend_irecv(ops) if ops else []
        if not self.is_async:
            for w in works:
                w.wait()
            return None
        return _Handles(works)


def _cast(src: torch.Tensor, dst: torch.Tensor) -> None:
    """fp32 <-> bf16 buffer copy (communicator.py:128,137) through the C ABI; CUDA tensors only."""
    _lib.require_cuda(src, dst)
    n = src.numel()
    if n == 0:
        return
    lib = _lib.lib()
    if src.dtype == torch.float32:
        rc = lib.gnnagg_cast_f32_to_bf16(src.data_ptr(), dst.data_ptr(), n, _lib.stream_ptr(src.device))
    else:
        rc = lib.gnnagg_cast_bf16_to_f32(src.data_ptr(), dst.data_ptr(), n, _lib.stream_ptr(src.device))
    _lib.check(rc, "cast")


class _CastAfter(object):
    def __init__(self, work, src, dst):
        self.work, self.src, self.dst = work, src, dst

    def wait(self):
        if self.work is not None:
            self.work.wait()
        rec = TimeRecorder.ctx
        t = rec.start() if rec else None
        _cast(self.src, self.dst)
        if rec:
            rec.record_dequantization_time(t)
