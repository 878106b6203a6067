import torch

from .CommSplits import CommSplits


def _prefix(splits, device):
    out = torch.zeros(len(splits) + 1, dtype=torch.int32)
    out[1:] = torch.tensor(splits, dtype=torch.int32).cumsum(0) if len(splits) else 0
    return out.to(device)


class CommBuffer(object):
    """fp32 (and, for 16-bit mode, bf16) send / receive buffers of the halo exchange, allocated
    once for the widest layer and reshaped per layer (data_manager/CommBuffer.py:4-25)."""

    def __init__(self, comm_splits: CommSplits, feat_len: int, bits: int, device=None, lean: bool = False,
                 plan=None) -> None:
        """lean (an addition, packed halo modes only): the fp32 staging buffers get a shape but no
        memory (meta tensors).  The fused pack and unpack paths of the Aggregator never touch them; at
        10^7 halo rows x 256 columns they would be tens of GB each.
        plan (an addition): a peer.PushPlan -- the buffers are then views into its peer-visible
        allocation, so that other ranks can store their rows straight into them."""
        size_send_buf = (sum(comm_splits.send_splits), feat_len)
        size_recv_buf = (sum(comm_splits.recv_splits), feat_len)
        self.lean = bool(lean) and bits in (2, 4, 8)
        buf_device = "meta" if self.lean else device
        if plan is not None and not self.lean:
            # no zero fill here: the allocation was zeroed before its address was published, and from then
            # on a peer's rows may arrive at any time
            self.send_buf = plan.region("send_buf", size_send_buf, torch.float32)
            self.recv_buf = plan.region("recv_buf", size_recv_buf, torch.float32)
        else:
            self.send_buf = torch.zeros(size_send_buf, dtype=torch.float32, device=buf_device)
            self.recv_buf = torch.zeros(size_recv_buf, dtype=torch.float32, device=buf_device)
        self.send_buf_fp16 = None
        self.recv_buf_fp16 = None
        if bits == 16:
            self.send_buf_fp16 = torch.zeros(size_send_buf, dtype=torch.bfloat16, device=device)
            self.recv_buf_fp16 = torch.zeros(size_recv_buf, dtype=torch.bfloat16, device=device)

    def resize_buffer(self, comm_splits: CommSplits, feat_len: int, bits: int) -> None:
        size_send_buf = (sum(comm_splits.send_splits), feat_len)
        size_recv_buf = (sum(comm_splits.recv_splits), feat_len)
        self.send_buf.resize_(size_send_buf)
        self.recv_buf.resize_(size_recv_buf)
        if bits == 16 and self.send_buf_fp16 is not None and self.recv_buf_fp16 is not None:
            self.send_buf_fp16.resize_(size_send_buf)
            self.recv_buf_fp16.resize_(size_recv_buf)


class CommBufferForQuantization(object):
    """Packed code buffers, fp32 + bf16 parameter buffers and the per-peer row prefixes the codec
    kernels take (data_manager/CommBuffer.py:27-49; there for bits == 2 only)."""

    def __init__(self, comm_splits: CommSplits, feat_len: int, bits: int, device=None, plan=None) -> None:
        if bits in (2, 4, 8):
            n_send, n_recv = sum(comm_splits.send_splits), sum(comm_splits.recv_splits)

            def wire(name, shape, dtype):  # the buffers that receive rows from other ranks
                if plan is not None:
                    return plan.region(name, shape, dtype)  # zeroed before its address was published
                return torch.zeros(shape, dtype=dtype, device=device)

            self.quantized_send_data_buf = wire("q_send_data", (sum(comm_splits.send_splits_int2), feat_len), torch.uint8)
            self.quantized_recv_data_buf = wire("q_recv_data", (sum(comm_splits.recv_splits_int2), feat_len), torch.uint8)
            self.quantized_send_params_buf_fp32 = torch.zeros((n_send, 2), dtype=torch.float32, device=device)
            self.quantized_recv_params_buf_fp32 = torch.zeros((n_recv, 2), dtype=torch.float32, device=device)
            self.quantized_send_params_buf_bf16 = wire("q_send_params", (n_send, 2), torch.bfloat16)
            self.quantized_recv_params_buf_bf16 = wire("q_recv_params", (n_recv, 2), torch.bfloat16)
            self.quantized_work_range_per_proc = _prefix(comm_splits.send_splits, device)
            self.dequantized_work_range_per_proc = _prefix(comm_splits.recv_splits, device)

    def resize_buffer(self, comm_splits: CommSplits, feat_len: int, bits: int) -> None:
        if bits in (2, 4, 8):
            self.quantized_send_data_buf.resize_((sum(comm_splits.send_splits_int2), feat_len))
            self.quantized_recv_data_buf.resize_((sum(comm_splits.recv_splits_int2), feat_len))
