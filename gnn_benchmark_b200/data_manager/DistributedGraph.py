from typing import Optional

from torch import Tensor

from ..sparse import SparseTensor
from .CommBuffer import CommBuffer, CommBufferForQuantization
from .CommSplits import CommSplits


class DistributedGraph(object):
    """One rank's share of the graph, plain halo path (data_manager/DistributedGraph.py:8-33).

    Field names are the reference's; `idx_nodes_send_to_others_i32` and `scatter_adj_t` are
    additions the CUDA path derives once: the int32 copy of the send index and the
    (n_local x n_send) unit matrix whose accumulating SpMM is the deterministic form of
    grad.index_add_(0, idx_nodes_send_to_others, buf) (model/layers/aggregator.py:197-199)."""

    def __init__(
        self,
        local_adj_t: SparseTensor,
        remote_adj_t: SparseTensor,
        idx_nodes_send_to_others: Tensor,
        num_nodes_send_to_others: list,
        num_nodes_recv_from_others: list,
        in_degrees: Tensor,
        comm_splits: CommSplits,
        comm_buf: CommBuffer,
        comm_buf_for_quantization: Optional[CommBufferForQuantization],
    ) -> None:
        self.local_adj_t = local_adj_t
        self.remote_adj_t = remote_adj_t
        self.idx_nodes_send_to_others = idx_nodes_send_to_others
        self.num_nodes_send_to_others = num_nodes_send_to_others
        self.num_nodes_recv_from_others = num_nodes_recv_from_others
        self.in_degrees = in_degrees
        self.comm_splits = comm_splits
        self.comm_buf = comm_buf
        self.comm_buf_for_quantization = comm_buf_for_quantization
        self.idx_nodes_send_to_others_i32 = None
        self.scatter_adj_t = None


class DistributedGraphForPre(object):
    """One rank's share of the graph, pre/post-aggregation path (DistributedGraph.py:35-59)."""

    def __init__(
        self,
        local_adj_t: SparseTensor,
        adj_t_pre_post_aggr_from: SparseTensor,
        adj_t_pre_post_aggr_to: SparseTensor,
        pre_post_aggr_from_splits: list,
        pre_post_aggr_to_splits: list,
        in_degrees: Tensor,
        comm_splits: CommSplits,
        comm_buf: CommBuffer,
        comm_buf_for_quantization: Optional[CommBufferForQuantization],
    ) -> None:
        self.local_adj_t = local_adj_t
        self.adj_t_pre_post_aggr_from = adj_t_pre_post_aggr_from
        self.adj_t_pre_post_aggr_to = adj_t_pre_post_aggr_to
        self.pre_post_aggr_from_splits = pre_post_aggr_from_splits
        self.pre_post_aggr_to_splits = pre_post_aggr_to_splits
        self.in_degrees = in_degrees
        self.comm_splits = comm_splits
        self.comm_buf = comm_buf
        self.comm_buf_for_quantization = comm_buf_for_quantization
