"""Communication-plan construction for one rank, with the reference's class and method names.

The reference builds these plans with per-edge Python loops and `.item()` calls, and the pre/post
plan additionally peer by peer, masking the whole edge list once per peer and growing its result
lists with `torch.cat` (self_benchmark/a64fx/data_manager/DataProcessor.py:39-53, 133-326,
429-445).  Here a plan is ONE pass over the rank's remote edges for all peers at once: the owner of
every source comes from a `searchsorted` on the partition starts, one stable sort groups the edges
by owner, multiplicities and the pre/post decision are segment operations on composite
(owner, id) keys, and the per-peer pieces the reference returns are cut out of the grouped arrays
by their counts.  It runs on whatever device the edge lists live on (CPU or GPU) and produces the
same arrays: halo slot numbering, per-peer split counts, send index, and the three sparse matrices
of the pre/post-aggregation scheme.  The stage functions the reference's unit tests call keep their
names and signatures and are thin adapters over the same pass.
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


def _prefix(counts: torch.Tensor) -> torch.Tensor:
    """[0, cumsum(counts)] as a CPU int64 tensor (the reference keeps its edge offsets on the host)."""
    out = torch.zeros(counts.numel() + 1, dtype=torch.int64)
    out[1:] = torch.cumsum(counts.to(torch.int64).cpu(), 0)
    return out


class DataProcessor(object):
    def __init__(self) -> None:
        pass

    @staticmethod
    def get_in_degrees(local_edges_list, remote_edges_list, num_local_nodes):
        """In-degree of every local node over local and remote in-edges, clamped to >= 1, (n,1)
        fp32 (DataProcessor.py:11-18): one histogram of all destination ids."""
        dst = torch.cat((local_edges_list[1].reshape(-1), remote_edges_list[1].reshape(-1)))
        degs = torch.bincount(dst, minlength=num_local_nodes)[:num_local_nodes]
        return degs.clamp_(min=1).to(torch.float32).unsqueeze(-1)

    @staticmethod
    def sort_remote_edges_list_based_on_remote_nodes(remote_edges_list):
        """Sort remote edges by (global) source id, in place (DataProcessor.py:20-26)."""
        sort_index = torch.sort(remote_edges_list[0], stable=True)[1]
        remote_edges_list[0], remote_edges_list[1] = remote_edges_list[0][sort_index], remote_edges_list[1][sort_index]
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


# ---- the one-pass engine of the pre/post plan --------------------------------------------------------
def _multiplicity(key: torch.Tensor) -> torch.Tensor:
    """For every element, how many times its value occurs in `key`."""
    if key.numel() == 0:
        return torch.zeros(0, dtype=torch.int64, device=key.device)
    _, inverse, counts = torch.unique(key, return_inverse=True, return_counts=True)
    return counts[inverse]


def _mask_of(idx: torch.Tensor, n: int) -> torch.Tensor:
    """Boolean mask of length n from either a boolean mask or a list of positions."""
    if idx.dtype == torch.bool:
        return idx
    m = torch.zeros(n, dtype=torch.bool, device=idx.device)
    m[idx.to(torch.int64)] = True
    return m


class _Grouped(object):
    """Pairs (first, second) of all peers, grouped by peer: `counts[p]` pairs belong to peer p."""

    def __init__(self, first, second, counts, distinct):
        self.first, self.second, self.counts, self.distinct = first, second, counts, distinct

    def per_peer(self):
        sizes = [int(c) for c in self.counts.tolist()]
        return list(zip(torch.split(self.first, sizes), torch.split(self.second, sizes)))


def _group_pairs(first, second, owner, sort_by_second: bool, span: int, world_size: int) -> _Grouped:
    """Order pairs by (owner, key) with key = second or first; pairs with equal (owner, key) keep their
    input order.  `distinct[p]` = number of different keys inside peer p = rows on the wire."""
    key = owner * span + (second if sort_by_second else first)
    key, perm = torch.sort(key, stable=True)
    counts = torch.bincount(owner, minlength=world_size)[:world_size] if owner.numel() else \
        torch.zeros(world_size, dtype=torch.int64, device=first.device)
    if key.numel():
        distinct = torch.bincount(torch.unique_consecutive(key) // span, minlength=world_size)[:world_size]
    else:
        distinct = torch.zeros(world_size, dtype=torch.int64, device=first.device)
    return _Grouped(first[perm], second[perm], counts, distinct)


def _ship_and_aggregate(src, dst, owner, post, span: int, world_size: int):
    """From the classified remote edges of all peers build, grouped by peer,
      * what each owner must learn (DataProcessor.py:250-279): the pre edges (s, d) plus (s, s) for
        every distinct post source, ordered by the second key;
      * what is aggregated here after the exchange (DataProcessor.py:281-326): the post edges (s, d)
        plus (d, d) for every distinct pre destination, ordered by the first key."""
    pre = ~post
    # distinct post sources / pre destinations of every peer, with their owners, from composite keys
    k_post = torch.unique(owner[post] * span + src[post])
    post_src, post_src_owner = k_post % span, k_post // span
    k_pre = torch.unique(owner[pre] * span + dst[pre])
    pre_dst, pre_dst_owner = k_pre % span, k_pre // span
    shipped = _group_pairs(torch.cat((src[pre], post_src)), torch.cat((dst[pre], post_src)),
                           torch.cat((owner[pre], post_src_owner)), True, span, world_size)
    aggregated = _group_pairs(torch.cat((src[post], pre_dst)), torch.cat((dst[post], pre_dst)),
                              torch.cat((owner[post], pre_dst_owner)), False, span, world_size)
    return shipped, aggregated


def _span(*tensors) -> int:
    m = 0
    for t in tensors:
        if t.numel():
            m = max(m, int(t.max()))
    return m + 1


def _classify(src, dst, owner, span: int) -> torch.Tensor:
    """post[e] = outdeg(src[e]) > indeg(dst[e]), both counted inside the edge's own peer subset
    (DataProcessor.py:227-248)."""
    return _multiplicity(owner * span + src) > _multiplicity(owner * span + dst)


def _plan_all_peers(begin_node_on_each_subgraph, src, dst, world_size: int):
    dev = src.device
    begin = torch.as_tensor(begin_node_on_each_subgraph, dtype=torch.int64, device=dev)
    owner = torch.searchsorted(begin, src, right=True) - 1
    inside = (owner >= 0) & (owner < world_size)  # sources outside every range belong to no peer
    if not bool(inside.all()):
        src, dst, owner = src[inside], dst[inside], owner[inside]
    owner, order = torch.sort(owner, stable=True)  # peers in order, edge order kept inside a peer
    src, dst = src[order], dst[order]
    span = _span(src, dst)
    post = _classify(src, dst, owner, span)
    return _ship_and_aggregate(src, dst, owner, post, span, world_size)


class DataProcessorForPreAggresive(object):
    def __init__(self) -> None:
        pass

    @staticmethod
    def get_degrees(nodes_list):
        """{node id: multiplicity} (DataProcessor.py:125-131); for small inputs and tests, the plan
        itself counts with `_multiplicity`."""
        unique_nodes_list, counts = torch.unique(nodes_list, return_counts=True)
        return dict(zip(unique_nodes_list.tolist(), counts.tolist()))

    @staticmethod
    def decide_pre_or_post_aggr(src_in_remote_edges, dst_in_remote_edges, is_pre, is_post):
        """Flags of one peer's edge subset: is_post where outdeg(s) > indeg(d), else is_pre."""
        n = src_in_remote_edges.shape[0]
        owner = torch.zeros(n, dtype=torch.int64, device=src_in_remote_edges.device)
        post = _classify(src_in_remote_edges, dst_in_remote_edges, owner, _span(src_in_remote_edges, dst_in_remote_edges))
        return torch.where(post, int(is_post), int(is_pre)).to(torch.int64)

    @staticmethod
    def _one_peer(src, dst, pre_aggr_edge_idx, post_aggr_edge_idx):
        n = src.shape[0]
        post = _mask_of(post_aggr_edge_idx, n)
        keep = post | _mask_of(pre_aggr_edge_idx, n)  # the caller's two selections, whatever made them
        src, dst, post = src[keep], dst[keep], post[keep]
        owner = torch.zeros(src.shape[0], dtype=torch.int64, device=src.device)
        return _ship_and_aggregate(src, dst, owner, post, _span(src, dst), 1)

    @staticmethod
    def collect_edges_sent_to_other_subgraphs(src_in_remote_edges, dst_in_remote_edges, pre_aggr_edge_idx,
                                              post_aggr_edge_idx, remote_edges_sent_for_graph_exchange):
        """Append one peer's shipped list [firsts..., seconds...] (DataProcessor.py:250-279)."""
        shipped, _ = DataProcessorForPreAggresive._one_peer(src_in_remote_edges, dst_in_remote_edges,
                                                            pre_aggr_edge_idx, post_aggr_edge_idx)
        remote_edges_sent_for_graph_exchange.append(torch.cat((shipped.first, shipped.second)))

    @staticmethod
    def collect_edges_for_aggregation(src_in_remote_edges, dst_in_remote_edges, pre_aggr_edge_idx, post_aggr_edge_idx,
                                      remote_edges_for_aggr_on_recv, recv_splits_for_data_exchange,
                                      begin_edge_on_each_partition_from, cur_rank):
        """Append one peer's receiver-side aggregation list, its receive split and its edge offset
        (DataProcessor.py:281-326)."""
        _, aggregated = DataProcessorForPreAggresive._one_peer(src_in_remote_edges, dst_in_remote_edges,
                                                               pre_aggr_edge_idx, post_aggr_edge_idx)
        recv_splits_for_data_exchange.append(int(aggregated.distinct[0]))
        remote_edges_for_aggr_on_recv[0] = torch.cat((remote_edges_for_aggr_on_recv[0], aggregated.first))
        remote_edges_for_aggr_on_recv[1] = torch.cat((remote_edges_for_aggr_on_recv[1], aggregated.second))
        begin_edge_on_each_partition_from[cur_rank + 1] = (begin_edge_on_each_partition_from[cur_rank]
                                                           + aggregated.first.shape[0])

    @staticmethod
    def split_remote_edges_for_aggr_and_graph_exchange(begin_node_on_each_subgraph, remote_edges_list, world_size):
        """All peers at once (DataProcessor.py:133-199): the shipped list of every peer, the
        receiver-side aggregation list (peers concatenated), its per-peer edge offsets and the receive
        splits."""
        shipped, aggregated = _plan_all_peers(begin_node_on_each_subgraph, remote_edges_list[0], remote_edges_list[1],
                                              world_size)
        sent = [torch.cat(pair) for pair in shipped.per_peer()]
        return (sent, [aggregated.first, aggregated.second], _prefix(aggregated.counts),
                [int(x) for x in aggregated.distinct.tolist()])

    @staticmethod
    def split_remote_edges_recv_from_graph_exchange(remote_edges_recv_from_graph_exchange, world_size):
        """Sender side (DataProcessor.py:201-225): every peer's message is [firsts..., seconds...];
        the rows this rank sends to that peer are its distinct second keys."""
        msgs = list(remote_edges_recv_from_graph_exchange)[:world_size]
        halves = [int(m.shape[0]) // 2 for m in msgs]
        dev = msgs[0].device if msgs else None
        empty = torch.empty(0, dtype=torch.int64, device=dev)
        first = torch.cat([m[:h] for m, h in zip(msgs, halves)]) if msgs else empty
        second = torch.cat([m[h:2 * h] for m, h in zip(msgs, halves)]) if msgs else empty
        counts = torch.tensor(halves, dtype=torch.int64)
        peer = torch.repeat_interleave(torch.arange(len(msgs), device=dev), counts.to(dev)) if msgs else empty
        if second.numel():
            span = _span(second)
            distinct = torch.bincount(torch.unique(peer * span + second) // span, minlength=world_size)[:world_size]
            send_splits = [int(x) for x in distinct.tolist()]
        else:
            send_splits = [0] * world_size
        return [first, second], _prefix(counts), send_splits

    @staticmethod
    def communicate_to_get_num_remote_edges(remote_edges_sent_for_graph_exchange, world_size):
        """Exchange the lengths of the shipped lists (DataProcessor.py:328-350)."""
        dev = remote_edges_sent_for_graph_exchange[0].device
        lengths = torch.tensor([t.shape[0] for t in remote_edges_sent_for_graph_exchange], dtype=torch.int64, device=dev)
        return lengths, (_exchange_counts(lengths, world_size) if world_size != 1 else torch.zeros_like(lengths))

    @staticmethod
    def communicate_to_get_remote_edges(remote_edges_sent_for_graph_exchange, send_splits_for_graph_exchange,
                                        recv_splits_for_graph_exchange, world_size):
        """Exchange the shipped lists themselves (DataProcessor.py:352-382)."""
        send_splits = [int(x) for x in send_splits_for_graph_exchange.tolist()]
        recv_splits = [int(x) for x in recv_splits_for_graph_exchange.tolist()]
        send = torch.cat(remote_edges_sent_for_graph_exchange)
        if world_size != 1:
            recv = _all_to_all_v(send, send_splits, recv_splits)
        else:
            recv = torch.empty(sum(recv_splits), dtype=torch.int64, device=send.device)
        return torch.split(recv, recv_splits)

    @staticmethod
    def divide_remote_edges_list(begin_node_on_each_subgraph, remote_edges_list, world_size):
        """Both sides of the pre/post plan of this rank (DataProcessor.py:384-427): classify and group
        locally, ship to the owners, regroup what the others shipped."""
        cls = DataProcessorForPreAggresive
        sent, for_recv, begin_from, recv_splits = cls.split_remote_edges_for_aggr_and_graph_exchange(
            begin_node_on_each_subgraph, remote_edges_list, world_size)
        n_send, n_recv = cls.communicate_to_get_num_remote_edges(sent, world_size)
        got = cls.communicate_to_get_remote_edges(sent, n_send, n_recv, world_size)
        for_send, begin_to, send_splits = cls.split_remote_edges_recv_from_graph_exchange(got, world_size)
        return for_recv, for_send, begin_from, begin_to, recv_splits, send_splits

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
        remap = DataProcessorForPreAggresive.remap_remote_nodes_id
        n = num_local_nodes
        local_adj_t = SparseTensor(row=local_edges_list[1], col=local_edges_list[0], sparse_sizes=(n, n))
        slot_from, dst_local = remote_edges_list_pre_post_aggr_from
        dst_local -= local_node_begin_idx
        num_slots_from = remap(slot_from, begin_edge_on_each_partition_from)  # keys -> slot ids, in place
        adj_t_pre_post_aggr_from = SparseTensor(row=dst_local, col=slot_from, sparse_sizes=(n, num_slots_from))
        src_local, slot_to = remote_edges_list_pre_post_aggr_to
        src_local -= local_node_begin_idx
        num_slots_to = remap(slot_to, begin_edge_on_each_partition_to)
        adj_t_pre_post_aggr_to = SparseTensor(row=slot_to, col=src_local, sparse_sizes=(num_slots_to, n))
        return local_adj_t, adj_t_pre_post_aggr_from, adj_t_pre_post_aggr_to
