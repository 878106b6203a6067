"""On-disk partition format (data_manager/DataLoader.py:12-61 of the reference): files written by
graphgen.write_partition_files are read back by load_data on 2 gloo ranks and give the same
DistributedGraph as the in-memory path."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _worker(rank, P, port, root, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen, load_data
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    Communicator(32)
    Quantizer_for_all_procs(P, 32)
    TimeRecorder(1, 1)
    ok = []
    n = 600
    src, dst = graphgen.erdos_renyi_edges(n, 2400, seed=3)
    src, dst = graphgen.symmetrize(src, dst, n, self_loops=True)
    begin = graphgen.contiguous_partitions(n, P)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    g = torch.Generator().manual_seed(rank)
    feat = torch.randn(b1 - b0, 12, generator=g)
    label = torch.randint(0, 5, (b1 - b0,), generator=g)
    perm = torch.randperm(b1 - b0, generator=g)
    part_dir = os.path.join(root, f"toy_{P}_part")
    graphgen.write_partition_files(part_dir, "toy", rank, begin, local, remote, feat, label, perm[:100], perm[100:150],
                                   perm[150:200])
    dist.barrier()
    for is_pre in (False, True):
        cfg = dict(input_dir=part_dir, graph_name="toy", num_bits=32, is_pre_delay=is_pre, in_channels=12,
                   hidden_channels=16, out_channels=5, device="cpu")
        data = load_data(cfg)
        ref = build_graph(local, remote, begin, rank, P, 16, 32, is_pre, device="cpu")
        gr = data["graph"]
        ok.append(torch.equal(data["nodes_features"], feat) and torch.equal(data["nodes_labels"], label))
        ok.append(torch.equal(data["nodes_train_masks"], perm[:100]) and data["nodes_test_masks"].numel() == 50)
        ok.append(gr.comm_splits.recv_splits == ref.comm_splits.recv_splits
                  and gr.comm_splits.send_splits == ref.comm_splits.send_splits)
        ok.append(torch.equal(gr.in_degrees, ref.in_degrees))
        for name in (("local_adj_t", "adj_t_pre_post_aggr_from", "adj_t_pre_post_aggr_to") if is_pre
                     else ("local_adj_t", "remote_adj_t")):
            a, b = getattr(gr, name), getattr(ref, name)
            ok.append(a.sparse_sizes() == b.sparse_sizes() and all(torch.equal(x, y) for x, y in zip(a.csr(), b.csr())))
        ok.append(gr.comm_buf.send_buf.shape == (sum(gr.comm_splits.send_splits), 16))
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(str(all(ok)) + " " + str(ok))
    dist.barrier()
    dist.destroy_process_group()


def test_write_then_load_data_matches_in_memory_plan(tmp_path):
    P = 2
    port = 29950 + (os.getpid() % 40)
    mp.spawn(_worker, args=(P, port, str(tmp_path), str(tmp_path)), nprocs=P, join=True)
    for r in range(P):
        msg = open(os.path.join(str(tmp_path), f"r{r}.txt")).read()
        assert msg.startswith("True"), f"rank {r}: {msg}"
