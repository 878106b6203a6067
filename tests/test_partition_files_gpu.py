"""load_data on the device path: the reference's per-rank partition files (written by
graphgen.write_partition_files) are loaded by 3 ranks whose plan exchange runs on CUDA tensors (the branch
load_data takes under NCCL: edge lists on the device, plan built there, graph validated by the library's
CSR check), and one aggregation over the loaded graph equals the one over the in-memory graph."""
import os
from types import SimpleNamespace

import numpy as np
import pytest
import torch

from fake_dist import FakeWorld

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("is_pre,bits", [(False, 32), (True, 32), (False, 2)])
def test_load_data_on_device_matches_in_memory_plan(cuda_lib, tmp_path, is_pre, bits):
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen, load_data
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    P, n, F = 3, 900, 12
    src, dst = graphgen.erdos_renyi_edges(n, 3600, seed=3)
    src, dst = graphgen.symmetrize(src, dst, n, self_loops=True)
    begin = graphgen.contiguous_partitions(n, P)
    part_dir = os.path.join(str(tmp_path), f"toy_{P}_part")
    feats, parts = [], []
    for rank in range(P):
        local, remote = graphgen.partition_edges(src, dst, begin, rank)
        b0, b1 = int(begin[rank]), int(begin[rank + 1])
        g = torch.Generator().manual_seed(rank)
        feat = torch.randn(b1 - b0, F, generator=g)
        label = torch.randint(0, 5, (b1 - b0,), generator=g)
        perm = torch.randperm(b1 - b0, generator=g)
        graphgen.write_partition_files(part_dir, "toy", rank, begin, local, remote, feat, label, perm[:100], perm[100:150],
                                       perm[150:200])
        feats.append(feat)
        parts.append((local, remote))
    Communicator(bits, is_async=True)
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(1, 1)

    def rank_fn(rank):
        cfg = dict(input_dir=part_dir, graph_name="toy", num_bits=bits, is_pre_delay=is_pre, in_channels=F,
                   hidden_channels=16, out_channels=5)  # no "device": the current CUDA device, plan built on it
        data = load_data(cfg)
        gr = data["graph"]
        local, remote = parts[rank]
        ref = build_graph(local.cuda(), remote.cuda(), begin, rank, P, 16, bits, is_pre, device="cuda")
        same = [gr.comm_splits.recv_splits == ref.comm_splits.recv_splits,
                gr.comm_splits.send_splits == ref.comm_splits.send_splits,
                torch.equal(gr.in_degrees, ref.in_degrees), data["nodes_features"].is_cuda,
                torch.equal(data["nodes_features"].cpu(), feats[rank])]
        for name in (("local_adj_t", "adj_t_pre_post_aggr_from", "adj_t_pre_post_aggr_to") if is_pre
                     else ("local_adj_t", "remote_adj_t")):
            a, b = getattr(gr, name), getattr(ref, name)
            same.append(a.sparse_sizes() == b.sparse_sizes() and a.device.type == "cuda"
                        and all(torch.equal(x, y) for x, y in zip(a.csr(), b.csr())))
        outs = []
        for graph in (gr, ref):
            ctx = SimpleNamespace()
            outs.append(Aggregator.forward(ctx, graph, data["nodes_features"], 0, bits, is_pre, True).cpu())
        same.append(torch.equal(outs[0], outs[1]))
        return same

    for r, same in enumerate(FakeWorld(P).run(rank_fn)):
        assert all(same), f"rank {r}: {same}"
