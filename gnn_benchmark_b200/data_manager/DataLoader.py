"""Per-rank partition loading and DistributedGraph assembly (reference:
self_benchmark/a64fx/data_manager/DataLoader.py:12-257).

On-disk format, per rank r in `<input_dir>`:
  p%03d-<graph>_nodes.npy         (n,2) int64 [new id, original id]; only [0][0], [-1][0] are read
  p%03d-<graph>_local_edges.npy   (2,E_l) int64 [src, dst], both local ids
  p%03d-<graph>_remote_edges.npy  (2,E_r) int64 [global src, local dst]
  p%03d-<graph>_nodes_feat.npy    (n,F) fp32;  _nodes_label.npy (n) int64
  p%03d-<graph>_nodes_{train,valid,test}_idx.npy  int64 local indices
  begin_node_on_each_partition.txt  one line, P+1 integers
"""
import os

import numpy as np
import torch
import torch.distributed as dist

from ..sparse import SparseTensor
from .CommBuffer import CommBuffer, CommBufferForQuantization
from .CommSplits import CommSplits
from .DataProcessor import DataProcessor, DataProcessorForPreAggresive
from .DistributedGraph import DistributedGraph, DistributedGraphForPre


def _part_file(input_dir, rank, graph_name, what):
    return os.path.join(input_dir, "p{:0>3d}-{}_{}.npy".format(rank, graph_name, what))


def load_graph_structures(input_dir, graph_name, rank):
    local_nodes_list = np.load(_part_file(input_dir, rank, graph_name, "nodes"))
    node_idx_begin = local_nodes_list[0][0]
    node_idx_end = local_nodes_list[local_nodes_list.shape[0] - 1][0]
    num_local_nodes = int(node_idx_end - node_idx_begin + 1)
    local_edges_list = np.load(_part_file(input_dir, rank, graph_name, "local_edges"))
    remote_edges_list = np.load(_part_file(input_dir, rank, graph_name, "remote_edges"))
    nodes_range_on_each_subgraph = np.loadtxt(
        os.path.join(input_dir, "begin_node_on_each_partition.txt"), dtype=np.int64, delimiter=" "
    )
    return (
        torch.from_numpy(local_nodes_list),
        torch.from_numpy(local_edges_list),
        torch.from_numpy(remote_edges_list),
        torch.from_numpy(nodes_range_on_each_subgraph),
        num_local_nodes,
    )


def load_nodes_labels(input_dir, graph_name, rank):
    return torch.from_numpy(np.load(_part_file(input_dir, rank, graph_name, "nodes_label")))


def load_nodes_features(input_dir, graph_name, rank):
    return torch.from_numpy(np.load(_part_file(input_dir, rank, graph_name, "nodes_feat")))


def load_dataset_mask(input_dir, graph_name, rank):
    return tuple(torch.from_numpy(np.load(_part_file(input_dir, rank, graph_name, f"nodes_{k}_idx")))
                 for k in ("train", "valid", "test"))


def pad_feature_rows(feat: torch.Tensor, multiple: int = 32) -> torch.Tensor:
    """The same (n, F) values as a view into rows of ceil(F / multiple) * multiple floats, so that every
    feature row starts on a 128-byte line of HBM (the aggregation gathers whole rows)."""
    n, f = feat.shape
    if f % multiple == 0:
        return feat.contiguous()
    store = torch.zeros(n, (f + multiple - 1) // multiple * multiple, dtype=feat.dtype, device=feat.device)
    store[:, :f] = feat
    return store[:, :f]


def _scatter_matrix(idx: torch.Tensor, num_local_nodes: int) -> SparseTensor:
    """(n_local x n_send) unit matrix S with S[idx[i], i] = 1: grad += S @ buf is
    grad.index_add_(0, idx, buf) with the additions of a row applied in increasing i."""
    cols = torch.arange(idx.numel(), dtype=torch.int64, device=idx.device)
    return SparseTensor(row=idx.to(torch.int64), col=cols, sparse_sizes=(num_local_nodes, idx.numel()))


def _push_plan(comm_splits, max_feat_len, bits, lean_halo, world_size):
    """The peer-visible receive buffers of this graph when the Communicator exchanges by direct stores
    (Communicator(transport="push")); None for the all-to-all transport."""
    from ..communicator import Communicator

    comm = Communicator.ctx
    if comm is None or world_size < 2 or getattr(comm, "transport", "all_to_all") != "push":
        return None
    from ..peer import PushPlan

    return PushPlan(comm.peers(), comm_splits, max_feat_len, bits, bool(lean_halo) and bits in (2, 4, 8))


def _check_graph(graph) -> None:
    """Refuse a malformed graph before any kernel runs on it: the gather, SpMM and codec kernels index
    device memory with these arrays and do no bounds checks of their own.  Every matrix goes through
    the device-side CSR check (row pointers monotone, columns in range); the send index must address
    local rows; the halo matrices must have exactly one column (row) per exchanged row.  CUDA graphs
    only: the check is a kernel of the library."""
    n = graph.local_adj_t.sparse_size(0)
    if not graph.local_adj_t.device.type == "cuda":
        return
    n_recv, n_send = sum(graph.comm_splits.recv_splits), sum(graph.comm_splits.send_splits)
    graph.local_adj_t.validate()
    if hasattr(graph, "remote_adj_t"):
        graph.remote_adj_t.validate()
        if graph.remote_adj_t.sparse_size(1) != n_recv or graph.remote_adj_t.sparse_size(0) != n:
            raise RuntimeError("remote_adj_t does not match the receive splits")
        idx = graph.idx_nodes_send_to_others
        if idx.numel() != n_send:
            raise RuntimeError("idx_nodes_send_to_others does not match the send splits")
        if idx.numel() and (int(idx.min()) < 0 or int(idx.max()) >= n):
            raise RuntimeError("idx_nodes_send_to_others addresses rows outside this partition")
        graph.scatter_adj_t.validate()
    else:
        graph.adj_t_pre_post_aggr_from.validate()
        graph.adj_t_pre_post_aggr_to.validate()
        if graph.adj_t_pre_post_aggr_from.sparse_sizes() != (n, n_recv) or \
                graph.adj_t_pre_post_aggr_to.sparse_sizes() != (n_send, n):
            raise RuntimeError("pre/post aggregation matrices do not match the exchange splits")
    q = graph.comm_buf_for_quantization
    if q is not None:
        if int(q.quantized_work_range_per_proc[-1]) != n_send or int(q.dequantized_work_range_per_proc[-1]) != n_recv:
            raise RuntimeError("per-peer row prefixes of the packed halo do not match the exchange splits")


def get_distributed_graph(local_edges_list, remote_edges_list, local_nodes_list, nodes_range_on_each_subgraph,
                          num_local_nodes: int, max_feat_len: int, world_size: int, bits: int, device=None,
                          lean_halo: bool = False):
    """Plain halo path (DataLoader.py:64-122).  Edge lists may live on CPU or GPU; the plan is
    built where they are and the resulting graph is moved to `device`."""
    in_degrees = DataProcessor.get_in_degrees(local_edges_list, remote_edges_list, num_local_nodes)
    remote_edges_list = DataProcessor.sort_remote_edges_list_based_on_remote_nodes(remote_edges_list)
    (
        remote_nodes_list,
        range_of_remote_nodes_on_local_graph,
        remote_nodes_num_from_each_subgraph,
    ) = DataProcessor.obtain_remote_nodes_list(remote_edges_list, num_local_nodes, nodes_range_on_each_subgraph,
                                               world_size)
    (
        local_nodes_required_by_other,
        num_local_nodes_required_by_other,
    ) = DataProcessor.obtain_local_nodes_required_by_other(
        local_nodes_list, remote_nodes_list, range_of_remote_nodes_on_local_graph,
        remote_nodes_num_from_each_subgraph, world_size,
    )
    local_adj_t, remote_adj_t = DataProcessor.transform_edge_index_to_sparse_tensor(
        local_edges_list, remote_edges_list, num_local_nodes, remote_nodes_list.size(0)
    )
    if device is None:
        device = local_adj_t.device
    comm_splits = CommSplits(remote_nodes_num_from_each_subgraph.tolist(),
                             num_local_nodes_required_by_other.tolist(), world_size, bits)
    plan = _push_plan(comm_splits, max_feat_len, bits, lean_halo, world_size)
    comm_buf = CommBuffer(comm_splits, max_feat_len, bits, device, lean=lean_halo, plan=plan)
    comm_buf_for_quantization = None
    if bits in (2, 4, 8):
        comm_buf_for_quantization = CommBufferForQuantization(comm_splits, max_feat_len, bits, device, plan=plan)
    graph = DistributedGraph(
        local_adj_t.to(device),
        remote_adj_t.to(device),
        local_nodes_required_by_other.to(device),
        num_local_nodes_required_by_other.tolist(),
        remote_nodes_num_from_each_subgraph.tolist(),
        in_degrees.to(device),
        comm_splits,
        comm_buf,
        comm_buf_for_quantization,
    )
    graph.idx_nodes_send_to_others_i32 = graph.idx_nodes_send_to_others.to(torch.int32)
    graph.scatter_adj_t = _scatter_matrix(graph.idx_nodes_send_to_others, num_local_nodes)
    graph.push_plan = plan
    _check_graph(graph)
    return graph


def get_distributed_graph_for_pre_aggressive(local_edges_list, remote_edges_list, nodes_range_on_each_subgraph,
                                             num_local_nodes, max_feat_len, rank, world_size, bits, device=None,
                                             lean_halo: bool = False):
    """Pre/post-aggregation path (DataLoader.py:125-194)."""
    in_degrees = DataProcessor.get_in_degrees(local_edges_list, remote_edges_list, num_local_nodes)
    # destinations back to global ids: pre/post keys mix ids of both ranks (DataLoader.py:139)
    remote_edges_list[1] += int(nodes_range_on_each_subgraph[rank])
    (
        remote_edges_list_pre_post_aggr_from,
        remote_edges_list_pre_post_aggr_to,
        begin_edge_on_each_partition_from,
        begin_edge_on_each_partition_to,
        pre_post_aggr_from_splits,
        pre_post_aggr_to_splits,
    ) = DataProcessorForPreAggresive.divide_remote_edges_list(nodes_range_on_each_subgraph, remote_edges_list,
                                                              world_size)
    (
        local_adj_t,
        adj_t_pre_post_aggr_from,
        adj_t_pre_post_aggr_to,
    ) = DataProcessorForPreAggresive.transform_edge_index_to_sparse_tensor(
        local_edges_list, remote_edges_list_pre_post_aggr_from, remote_edges_list_pre_post_aggr_to,
        begin_edge_on_each_partition_from, begin_edge_on_each_partition_to, num_local_nodes,
        int(nodes_range_on_each_subgraph[rank]),
    )
    if device is None:
        device = local_adj_t.device
    comm_splits = CommSplits(pre_post_aggr_from_splits, pre_post_aggr_to_splits, world_size, bits)
    plan = _push_plan(comm_splits, max_feat_len, bits, lean_halo, world_size)
    comm_buf = CommBuffer(comm_splits, max_feat_len, bits, device, lean=lean_halo, plan=plan)
    comm_buf_for_quantization = None
    if bits in (2, 4, 8):
        comm_buf_for_quantization = CommBufferForQuantization(comm_splits, max_feat_len, bits, device, plan=plan)
    graph = DistributedGraphForPre(
        local_adj_t.to(device),
        adj_t_pre_post_aggr_from.to(device),
        adj_t_pre_post_aggr_to.to(device),
        pre_post_aggr_from_splits,
        pre_post_aggr_to_splits,
        in_degrees.to(device),
        comm_splits,
        comm_buf,
        comm_buf_for_quantization,
    )
    graph.push_plan = plan
    _check_graph(graph)
    return graph


def build_graph(local_edges_list, remote_edges_list, nodes_range_on_each_subgraph, rank, world_size, max_feat_len,
                bits, is_pre_delay, device=None, lean_halo: bool = False):
    """Assemble a DistributedGraph[ForPre] from in-memory edge lists (what load_data does after
    reading the files).  local_edges_list / remote_edges_list: 2 x E int64 tensors or pairs."""
    local_edges_list = [local_edges_list[0], local_edges_list[1]]
    remote_edges_list = [remote_edges_list[0].clone(), remote_edges_list[1].clone()]
    begin = nodes_range_on_each_subgraph
    num_local_nodes = int(begin[rank + 1]) - int(begin[rank])
    if is_pre_delay:
        return get_distributed_graph_for_pre_aggressive(local_edges_list, remote_edges_list, begin, num_local_nodes,
                                                        max_feat_len, rank, world_size, bits, device,
                                                        lean_halo=lean_halo)
    local_nodes_list = torch.tensor([[int(begin[rank]), 0]], dtype=torch.int64)
    return get_distributed_graph(local_edges_list, remote_edges_list, local_nodes_list, begin, num_local_nodes,
                                 max_feat_len, world_size, bits, device, lean_halo=lean_halo)


def load_data(config):
    """Reference entry point (DataLoader.py:197-257): config keys input_dir, graph_name, num_bits,
    is_pre_delay, in_channels, hidden_channels, out_channels; optional `device` (default: the
    current CUDA device)."""
    input_dir = config["input_dir"]
    graph_name = config["graph_name"]
    num_bits = config["num_bits"]
    is_pre_delay = config["is_pre_delay"]
    rank = dist.get_rank()
    world_size = dist.get_world_size()
    max_feat_len = max(config["in_channels"], config["hidden_channels"], config["out_channels"])
    device = config.get("device")
    if device is None:
        device = torch.device("cuda", torch.cuda.current_device())
    device = torch.device(device)

    (
        local_nodes_list,
        local_edges_list,
        remote_edges_list,
        nodes_range_on_each_subgraph,
        num_local_nodes,
    ) = load_graph_structures(input_dir, graph_name, rank)
    # the collectives of the plan exchange need tensors the process group can move
    plan_device = device if dist.get_backend() == "nccl" else torch.device("cpu")
    local_edges_list = [local_edges_list[0].to(plan_device), local_edges_list[1].to(plan_device)]
    remote_edges_list = [remote_edges_list[0].to(plan_device), remote_edges_list[1].to(plan_device)]

    if is_pre_delay:
        distributed_graph = get_distributed_graph_for_pre_aggressive(
            local_edges_list, remote_edges_list, nodes_range_on_each_subgraph, num_local_nodes, max_feat_len, rank,
            world_size, num_bits, device)
    else:
        distributed_graph = get_distributed_graph(
            local_edges_list, remote_edges_list, local_nodes_list, nodes_range_on_each_subgraph, num_local_nodes,
            max_feat_len, world_size, num_bits, device)

    train_mask, valid_mask, test_mask = load_dataset_mask(input_dir, graph_name, rank)
    data = dict()
    data["graph"] = distributed_graph
    data["nodes_features"] = pad_feature_rows(load_nodes_features(input_dir, graph_name, rank).to(device))
    data["nodes_labels"] = load_nodes_labels(input_dir, graph_name, rank).to(device)
    data["nodes_train_masks"] = train_mask.to(device)
    data["nodes_valid_masks"] = valid_mask.to(device)
    data["nodes_test_masks"] = test_mask.to(device)
    return data
