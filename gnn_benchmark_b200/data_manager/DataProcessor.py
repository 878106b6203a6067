"""Communication-plan construction for one rank, with the reference's class and method names.

The reference builds these plans with per-edge Python loops and `.item()` calls
(self_benchmark/a64fx/data_manager/DataProcessor.py:39-53, 238-246, 438-444).  Here every
step is a sort / unique / searchsorted / cumsum over whole tensors, so it runs on whatever
device the edge lists live on (CPU or GPU) and scales to billions of edges, while producing
the same arrays: halo slot numbering, per-peer split counts, send index, and the three
sparse matrices of the pre/post-aggregation scheme.
"""
import torch
import torch.distributed as dist

from ..sparse import SparseTensor


def _all_to_all_v(send: torch.Tensor, send_splits, recv_splits) -> torch.Tensor:
    """all_to_all_single with per-peer element counts; works for CPU (gloo) and CUDA (nccl)."""
    recv = torch.empty(int(sum(recv_splits)), dtype=send.dtype, device=send.device)
    dist.all_to_all_single(recv, send.contiguous(), list(recv_splits), list(send_splits))
    return recv


def _exchange_counts(counts: torch.Tensor, world_size: int) -> torch.Tensor:
    counts = counts.to(torch.int64).contiguous()
    out = torch.zeros_like(counts)
    if world_size != 1:
        dist.all_to_all_single(out, counts, [1] * world_size, [1] * world_size)
    else:
        out.copy_(counts)
    return out


class DataProcessor(object):
    def __init__(self) -> None:
        pass

    @staticmethod
    def get_in_degrees(local_edges_list, remote_edges_list, num_local_nodes):
        """In-degree of every local node over local and remote in-edges, clamped to >= 1, (n,1)
        fp32 (DataProcessor.py:11-18)."""
        dev = local_edges_list[1].device
        local_degs = torch.zeros((num_local_nodes), dtype=torch.float32, device=dev)
        source = torch.ones((local_edges_list[1].shape[0]), dtype=torch.float32, device=dev)
        local_degs.index_add_(dim=0, index=local_edges_list[1], source=source)
        source = torch.ones((remote_edges_list[1].shape[0]), dtype=torch.float32, device=dev)
        local_degs.index_add_(dim=0, index=remote_edges_list[1], source=source)
        return local_degs.clamp(min=1).unsqueeze(-1)

    @staticmethod
    def sort_remote_edges_list_based_on_remote_nodes(remote_edges_list):
        """Sort remote edges by (global) source id, in place (DataProcessor.py:20-26)."""
        remote_edges_row, remote_edges_col = remote_edges_list[0], remote_edges_list[1]
        sort_index = torch.sort(remote_edges_row, stable=True)[1]
        remote_edges_list[0] = remote_edges_row[sort_index]
        remote_edges_list[1] = remote_edges_col[sort_index]
        return remote_edges_list

    @staticmethod
    def obtain_remote_nodes_list(remote_edges_list, num_local_nodes, num_nodes_on_each_subgraph, world_size):
        """Halo renumbering (DataProcessor.py:28-60).  Input: remote edges sorted by source.

        Returns the sorted unique remote sources, the prefix of their counts per owner rank
        (P+1) and the counts (P).  As in the reference, row 0 of remote_edges_list is rewritten
        in place to the halo slot id num_local_nodes + rank_of_source_in_unique_list."""
        remote_edges_row = remote_edges_list[0]
        dev = remote_edges_row.device
        begin = torch.as_tensor(num_nodes_on_each_subgraph, dtype=torch.int64, device=dev)
        if remote_edges_row.numel() == 0:
            remote_nodes_list = torch.zeros(0, dtype=torch.int64, device=dev)
            counts = torch.zeros(world_size, dtype=torch.int64, device=dev)
        else:
            remote_nodes_list, inverse = torch.unique_consecutive(remote_edges_row, return_inverse=True)
            owner = torch.searchsorted(begin, remote_nodes_list, right=True) - 1
            counts = torch.bincount(owner, minlength=world_size)[:world_size]
            remote_edges_row.copy_(inverse + num_local_nodes)
        rng = torch.zeros(world_size + 1, dtype=torch.int64, device=dev)
        torch.cumsum(counts, 0, out=rng[1:])
        return remote_nodes_list.to(torch.int64), rng, counts.to(torch.int64)

    @staticmethod
    def obtain_local_nodes_required_by_other(
        local_nodes_list,
        remote_nodes_list,
        range_of_remote_nodes_on_local_graph,
        remote_nodes_num_from_each_subgraph,
        world_size,
    ):
        """Tell every owner which of its nodes this rank needs; learn which local nodes the
        others need (DataProcessor.py:62-98).  The reference uses the list form of
        dist.all_to_all; the single-tensor form used here carries the same payload."""
        num_required = _exchange_counts(remote_nodes_num_from_each_subgraph, world_size)
        send_splits = [int(x) for x in remote_nodes_num_from_each_subgraph.tolist()]
        recv_splits = [int(x) for x in num_required.tolist()]
        if world_size != 1:
            recv_nodes = _all_to_all_v(remote_nodes_list, send_splits, recv_splits)
        else:
            recv_nodes = remote_nodes_list.clone()
        local_node_idx_begin = local_nodes_list[0][0]
        return recv_nodes - local_node_idx_begin, num_required

    @staticmethod
    def transform_edge_index_to_sparse_tensor(local_edges_list, remote_edges_list, num_local_nodes, num_remote_nodes):
        """local_adj_t (n x n) and remote_adj_t (n x n_halo), all values 1 (DataProcessor.py:100-118).
        Row = destination, column = source; remote sources are halo slots minus num_local_nodes."""
        local_adj_t = SparseTensor(row=local_edges_list[1], col=local_edges_list[0],
                                   sparse_sizes=(num_local_nodes, num_local_nodes))
        remote_adj_t = SparseTensor(row=remote_edges_list[1], col=remote_edges_list[0] - num_local_nodes,
                                    sparse_sizes=(num_local_nodes, num_remote_nodes))
        return local_adj_t, remote_adj_t


def _multiplicity(x: torch.Tensor) -> torch.Tensor:
    """For every element, how many times its value occurs in x."""
    if x.numel() == 0:
        return torch.zeros(0, dtype=torch.int64, device=x.device)
    _, inverse, counts = torch.unique(x, return_inverse=True, return_counts=True)
    return counts[inverse]


def _sort_pairs(first: torch.Tensor, second: torch.Tensor, by_second: bool):
    key = second if by_second else first
    idx = torch.sort(key, stable=True)[1]
    return first[idx], second[idx]


class DataProcessorForPreAggresive(object):
    def __init__(self) -> None:
        pass

    @staticmethod
    def get_degrees(nodes_list):
        """{node id: multiplicity} (DataProcessor.py:125-131); kept for small inputs and tests,
        the plan builder itself uses the tensor form `_multiplicity`."""
        unique_nodes_list, counts = torch.unique(nodes_list, return_counts=True)
        return dict(zip(unique_nodes_list.tolist(), counts.tolist()))

    @staticmethod
    def decide_pre_or_post_aggr(src_in_remote_edges, dst_in_remote_edges, is_pre, is_post):
        """Edge (s, d) is post-aggregated iff outdeg(s) > indeg(d) inside this peer's edge
        subset, else pre-aggregated (DataProcessor.py:227-248)."""
        out_deg = _multiplicity(src_in_remote_edges)
        in_deg = _multiplicity(dst_in_remote_edges)
        flags = torch.full((src_in_remote_edges.shape[0],), is_pre, dtype=torch.int64,
                           device=src_in_remote_edges.device)
        flags[out_deg > in_deg] = is_post
        return flags

    @staticmethod
    def collect_edges_sent_to_other_subgraphs(src_in_remote_edges, dst_in_remote_edges, pre_aggr_edge_idx,
                                              post_aggr_edge_idx, remote_edges_sent_for_graph_exchange):
        """What the owner of the sources must learn (DataProcessor.py:250-279): the pre edges
        (s, d) plus (s, s) for every unique post source, sorted by the second key, appended as
        one tensor [firsts..., seconds...]."""
        src_in_pre = src_in_remote_edges[pre_aggr_edge_idx]
        dst_in_pre = dst_in_remote_edges[pre_aggr_edge_idx]
        src_in_post = torch.unique(src_in_remote_edges[post_aggr_edge_idx], sorted=True)
        src_to_send = torch.cat((src_in_pre, src_in_post), dim=0)
        dst_to_send = torch.cat((dst_in_pre, src_in_post), dim=0)
        src_to_send, dst_to_send = _sort_pairs(src_to_send, dst_to_send, by_second=True)
        remote_edges_sent_for_graph_exchange.append(torch.cat((src_to_send, dst_to_send), dim=0))

    @staticmethod
    def collect_edges_for_aggregation(src_in_remote_edges, dst_in_remote_edges, pre_aggr_edge_idx, post_aggr_edge_idx,
                                      remote_edges_for_aggr_on_recv, recv_splits_for_data_exchange,
                                      begin_edge_on_each_partition_from, cur_rank):
        """Receiver-side aggregation list of one peer (DataProcessor.py:281-326): the post edges
        (s, d) plus (d, d) for every unique pre destination, sorted by the first key; the number
        of distinct first keys is this peer's receive split."""
        src_in_post = src_in_remote_edges[post_aggr_edge_idx]
        dst_in_post = dst_in_remote_edges[post_aggr_edge_idx]
        dst_in_pre = dst_in_remote_edges[pre_aggr_edge_idx]
        dst_from_recv = torch.unique(dst_in_pre, sorted=True)
        src_from_recv = torch.cat((src_in_post, dst_from_recv), dim=0)
        dst_from_recv = torch.cat((dst_in_post, dst_from_recv), dim=0)
        src_from_recv, dst_from_recv = _sort_pairs(src_from_recv, dst_from_recv, by_second=False)
        recv_splits_for_data_exchange.append(int(torch.unique(src_from_recv).shape[0]))
        remote_edges_for_aggr_on_recv[0] = torch.cat((remote_edges_for_aggr_on_recv[0], src_from_recv), dim=0)
        remote_edges_for_aggr_on_recv[1] = torch.cat((remote_edges_for_aggr_on_recv[1], dst_from_recv), dim=0)
        begin_edge_on_each_partition_from[cur_rank + 1] = (
            begin_edge_on_each_partition_from[cur_rank] + src_from_recv.shape[0]
        )

    @staticmethod
    def split_remote_edges_for_aggr_and_graph_exchange(begin_node_on_each_subgraph, remote_edges_list, world_size):
        """Per peer: classify its remote edges, build what is shipped to it and what is aggregated
        here (DataProcessor.py:133-199)."""
        dev = remote_edges_list[0].device
        remote_edges_sent_for_graph_exchange = []
        recv_splits_for_data_exchange = []
        begin_edge_on_each_partition_from = torch.zeros(world_size + 1, dtype=torch.int64)
        remote_edges_for_aggr_on_recv = [
            torch.empty((0), dtype=torch.int64, device=dev),
            torch.empty((0), dtype=torch.int64, device=dev),
        ]
        is_pre, is_post = 1, 0
        all_src, all_dst = remote_edges_list[0], remote_edges_list[1]
        for i in range(world_size):
            begin_idx = int(begin_node_on_each_subgraph[i])
            end_idx = int(begin_node_on_each_subgraph[i + 1])
            edge_idx = (all_src >= begin_idx) & (all_src < end_idx)
            src = all_src[edge_idx]
            dst = all_dst[edge_idx]
            flags = DataProcessorForPreAggresive.decide_pre_or_post_aggr(src, dst, is_pre, is_post)
            pre_aggr_edge_idx = flags == is_pre
            post_aggr_edge_idx = flags == is_post
            DataProcessorForPreAggresive.collect_edges_sent_to_other_subgraphs(
                src, dst, pre_aggr_edge_idx, post_aggr_edge_idx, remote_edges_sent_for_graph_exchange)
            DataProcessorForPreAggresive.collect_edges_for_aggregation(
                src, dst, pre_aggr_edge_idx, post_aggr_edge_idx, remote_edges_for_aggr_on_recv,
                recv_splits_for_data_exchange, begin_edge_on_each_partition_from, i)
        begin_edge_on_each_partition_from[world_size] = remote_edges_for_aggr_on_recv[0].shape[0]
        return (
            remote_edges_sent_for_graph_exchange,
            remote_edges_for_aggr_on_recv,
            begin_edge_on_each_partition_from,
            recv_splits_for_data_exchange,
        )

    @staticmethod
    def split_remote_edges_recv_from_graph_exchange(remote_edges_recv_from_graph_exchange, world_size):
        """Sender side: unpack what each peer shipped ([firsts..., seconds...]) and count the
        distinct second keys = rows this rank sends to that peer (DataProcessor.py:201-225)."""
        dev = remote_edges_recv_from_graph_exchange[0].device if len(remote_edges_recv_from_graph_exchange) else None
        remote_edges_for_aggr_for_send = [
            torch.empty((0), dtype=torch.int64, device=dev),
            torch.empty((0), dtype=torch.int64, device=dev),
        ]
        begin_edge_on_each_partition_to = torch.zeros(world_size + 1, dtype=torch.int64)
        send_splits_for_data_exchange = []
        for i in range(world_size):
            num_remote_edges = int(remote_edges_recv_from_graph_exchange[i].shape[0] / 2)
            src = remote_edges_recv_from_graph_exchange[i][:num_remote_edges]
            dst = remote_edges_recv_from_graph_exchange[i][num_remote_edges:]
            send_splits_for_data_exchange.append(int(torch.unique(dst).shape[0]))
            remote_edges_for_aggr_for_send[0] = torch.cat((remote_edges_for_aggr_for_send[0], src), dim=0)
            remote_edges_for_aggr_for_send[1] = torch.cat((remote_edges_for_aggr_for_send[1], dst), dim=0)
            begin_edge_on_each_partition_to[i + 1] = begin_edge_on_each_partition_to[i] + dst.shape[0]
        begin_edge_on_each_partition_to[world_size] = remote_edges_for_aggr_for_send[0].shape[0]
        return remote_edges_for_aggr_for_send, begin_edge_on_each_partition_to, send_splits_for_data_exchange

    @staticmethod
    def communicate_to_get_num_remote_edges(remote_edges_sent_for_graph_exchange, world_size):
        """Exchange the lengths of the shipped lists (DataProcessor.py:328-350)."""
        dev = remote_edges_sent_for_graph_exchange[0].device
        num_remote_edges_send = torch.tensor([t.shape[0] for t in remote_edges_sent_for_graph_exchange],
                                             dtype=torch.int64, device=dev)
        num_remote_edges_recv = torch.zeros(world_size, dtype=torch.int64, device=dev)
        if world_size != 1:
            dist.all_to_all_single(num_remote_edges_recv, num_remote_edges_send, [1] * world_size, [1] * world_size)
        return num_remote_edges_send, num_remote_edges_recv

    @staticmethod
    def communicate_to_get_remote_edges(remote_edges_sent_for_graph_exchange, send_splits_for_graph_exchange,
                                        recv_splits_for_graph_exchange, world_size):
        """Exchange the shipped lists themselves (DataProcessor.py:352-382)."""
        send_splits = [int(x) for x in send_splits_for_graph_exchange.tolist()]
        recv_splits = [int(x) for x in recv_splits_for_graph_exchange.tolist()]
        send = torch.cat(remote_edges_sent_for_graph_exchange, dim=0)
        recv = torch.empty(sum(recv_splits), dtype=torch.int64, device=send.device)
        if world_size != 1:
            dist.all_to_all_single(recv, send, recv_splits, send_splits)
        return torch.split(recv, recv_splits, dim=0)

    @staticmethod
    def divide_remote_edges_list(begin_node_on_each_subgraph, remote_edges_list, world_size):
        """DataProcessor.py:384-427."""
        (
            remote_edges_sent_for_graph_exchange,
            remote_edges_for_aggr_on_recv,
            begin_edge_on_each_partition_from,
            recv_splits_for_data_exchange,
        ) = DataProcessorForPreAggresive.split_remote_edges_for_aggr_and_graph_exchange(
            begin_node_on_each_subgraph, remote_edges_list, world_size
        )
        send_splits, recv_splits = DataProcessorForPreAggresive.communicate_to_get_num_remote_edges(
            remote_edges_sent_for_graph_exchange, world_size
        )
        remote_edges_recv_from_graph_exchange = DataProcessorForPreAggresive.communicate_to_get_remote_edges(
            remote_edges_sent_for_graph_exchange, send_splits, recv_splits, world_size
        )
        (
            remote_edges_for_aggr_for_send,
            begin_edge_on_each_partition_to,
            send_splits_for_data_exchange,
        ) = DataProcessorForPreAggresive.split_remote_edges_recv_from_graph_exchange(
            remote_edges_recv_from_graph_exchange, world_size
        )
        return (
            remote_edges_for_aggr_on_recv,
            remote_edges_for_aggr_for_send,
            begin_edge_on_each_partition_from,
            begin_edge_on_each_partition_to,
            recv_splits_for_data_exchange,
            send_splits_for_data_exchange,
        )

    @staticmethod
    def remap_remote_nodes_id(remote_nodes_list, begin_edge_on_each_partition):
        """Rewrite the (per-peer sorted) key list in place to consecutive wire-slot ids: a new id
        starts at every change of key and at every peer boundary (DataProcessor.py:429-445).
        Returns the number of slots."""
        n = int(begin_edge_on_each_partition[-1])
        if n == 0:
            return 0
        dev = remote_nodes_list.device
        keys = remote_nodes_list[:n]
        new_run = torch.ones(n, dtype=torch.bool, device=dev)
        new_run[1:] = keys[1:] != keys[:-1]
        starts = torch.as_tensor(begin_edge_on_each_partition, dtype=torch.int64, device=dev)[:-1]
        starts = starts[starts < n]
        new_run[starts] = True
        ids = torch.cumsum(new_run.to(torch.int64), 0) - 1
        remote_nodes_list[:n] = ids
        return int(ids[-1].item()) + 1

    @staticmethod
    def transform_edge_index_to_sparse_tensor(local_edges_list, remote_edges_list_pre_post_aggr_from,
                                              remote_edges_list_pre_post_aggr_to, begin_edge_on_each_partition_from,
                                              begin_edge_on_each_partition_to, num_local_nodes,
                                              local_node_begin_idx):
        """The three matrices of the pre/post scheme, all values 1 (DataProcessor.py:447-508):
        local_adj_t (n x n); adj_t_pre_post_aggr_from (n x recv slots): row = local destination,
        col = wire slot; adj_t_pre_post_aggr_to (send slots x n): row = wire slot, col = local
        source."""
        local_adj_t = SparseTensor(row=local_edges_list[1], col=local_edges_list[0],
                                   sparse_sizes=(num_local_nodes, num_local_nodes))
        remote_edges_list_pre_post_aggr_from[1] -= local_node_begin_idx
        num_remote_nodes_from = DataProcessorForPreAggresive.remap_remote_nodes_id(
            remote_edges_list_pre_post_aggr_from[0], begin_edge_on_each_partition_from
        )
        adj_t_pre_post_aggr_from = SparseTensor(
            row=remote_edges_list_pre_post_aggr_from[1], col=remote_edges_list_pre_post_aggr_from[0],
            sparse_sizes=(num_local_nodes, num_remote_nodes_from),
        )
        remote_edges_list_pre_post_aggr_to[0] -= local_node_begin_idx
        num_remote_nodes_to = DataProcessorForPreAggresive.remap_remote_nodes_id(
            remote_edges_list_pre_post_aggr_to[1], begin_edge_on_each_partition_to
        )
        adj_t_pre_post_aggr_to = SparseTensor(
            row=remote_edges_list_pre_post_aggr_to[1], col=remote_edges_list_pre_post_aggr_to[0],
            sparse_sizes=(num_remote_nodes_to, num_local_nodes),
        )
        return local_adj_t, adj_t_pre_post_aggr_from, adj_t_pre_post_aggr_to
