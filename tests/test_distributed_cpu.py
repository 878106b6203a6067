"""Host-side logic of the multi-rank path as real gloo processes on CPU (world sizes 2-5): the plan
exchange of both plan builders against the reference's golden plans, and the Communicator's fp32 halo
exchange in both directions.  No kernels run here (the compute path is CUDA-only)."""
import glob
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _keys(sp):
    rowptr, col, _ = sp.csr()
    rows = np.repeat(np.arange(sp.sparse_size(0)), np.diff(rowptr.numpy()))
    return rows * max(sp.sparse_size(1), 1) + col.numpy().astype(np.int64)


def _coo_keys(row, col, ncol):
    return np.sort(np.asarray(row, np.int64) * max(int(ncol), 1) + np.asarray(col, np.int64))


def _plan_worker(rank, P, port, plain_path, pre_path, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    Communicator(32, is_async=False)
    Quantizer_for_all_procs(P, 2)
    TimeRecorder(1, 1)
    problems = []
    try:
        g = np.load(plain_path)
        begin = torch.from_numpy(g["begin"])
        local = torch.from_numpy(g[f"r{rank}_local_edges"])
        remote = torch.from_numpy(g[f"r{rank}_remote_edges"])
        graph = build_graph(local, remote, begin, rank, P, 8, 2, False, device="cpu")
        n = int(begin[rank + 1] - begin[rank])
        checks = [
            (graph.comm_splits.recv_splits, g[f"r{rank}_recv_splits"].tolist(), "recv_splits"),
            (graph.comm_splits.send_splits, g[f"r{rank}_send_splits"].tolist(), "send_splits"),
            (graph.idx_nodes_send_to_others.tolist(), g[f"r{rank}_idx_nodes_send_to_others"].tolist(), "send idx"),
            (graph.in_degrees.numpy().tolist(), g[f"r{rank}_in_degrees"].tolist(), "in_degrees"),
            (_keys(graph.remote_adj_t).tolist(),
             _coo_keys(g[f"r{rank}_remote_row"], g[f"r{rank}_remote_col"], graph.remote_adj_t.sparse_size(1)).tolist(),
             "remote_adj_t"),
            (graph.comm_splits.recv_splits_int2, [-(-x // 4) for x in g[f"r{rank}_recv_splits"].tolist()], "int2 splits"),
            (graph.comm_buf_for_quantization.quantized_work_range_per_proc.tolist(),
             [0] + np.cumsum(g[f"r{rank}_send_splits"]).tolist(), "work range"),
        ]
        for got, want, name in checks:
            if got != want:
                problems.append(f"plain/{name}")
        # the scatter matrix is the transpose-gather of the send index
        s = graph.scatter_adj_t
        if s.sparse_sizes() != (n, len(graph.idx_nodes_send_to_others)):
            problems.append("scatter shape")

        # fp32 halo exchange, forward then backward (buffers and splits swap roles)
        from gnn_benchmark_b200 import Communicator as C
        F = 8
        graph.comm_buf.resize_buffer(graph.comm_splits, F, 32)
        X = torch.arange(int(begin[-1]) * F, dtype=torch.float32).view(-1, F)
        b0 = int(begin[rank])
        graph.comm_buf.send_buf.copy_(X[b0 + graph.idx_nodes_send_to_others])
        h = C.ctx.comm(graph.comm_splits, graph.comm_buf, None, "forward0", True, "forward")
        if h is not None:
            h.wait()
        want_rows = torch.from_numpy(g[f"r{rank}_remote_nodes_list"])
        if not torch.equal(graph.comm_buf.recv_buf, X[want_rows]):
            problems.append("forward halo rows")
        graph.comm_buf.recv_buf.mul_(2.0)
        h = C.ctx.comm(graph.comm_splits, graph.comm_buf, None, "backward0", True, "backward")
        if h is not None:
            h.wait()
        if not torch.equal(graph.comm_buf.send_buf, 2.0 * X[b0 + graph.idx_nodes_send_to_others]):
            problems.append("backward halo rows")

        g = np.load(pre_path)
        local = torch.from_numpy(g[f"r{rank}_local_edges"])
        remote = torch.from_numpy(g[f"r{rank}_remote_edges"])
        graph = build_graph(local, remote, begin, rank, P, 8, 32, True, device="cpu")
        if graph.pre_post_aggr_from_splits != g[f"r{rank}_recv_splits"].tolist():
            problems.append("pre/recv_splits")
        if graph.pre_post_aggr_to_splits != g[f"r{rank}_send_splits"].tolist():
            problems.append("pre/send_splits")
        if _keys(graph.adj_t_pre_post_aggr_from).tolist() != _coo_keys(g[f"r{rank}_from_row"], g[f"r{rank}_from_col"],
                                                                      int(g[f"r{rank}_n_from"])).tolist():
            problems.append("pre/adj_from")
        if _keys(graph.adj_t_pre_post_aggr_to).tolist() != _coo_keys(g[f"r{rank}_to_row"], g[f"r{rank}_to_col"],
                                                                    n).tolist():
            problems.append("pre/adj_to")
    except Exception as e:  # noqa: BLE001
        problems.append(f"exception: {e!r}")
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write("\n".join(problems))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("name", ["a", "b", "c", "d"])
def test_plan_exchange_and_halo_on_gloo(tmp_path, name):
    plain = os.path.join(GOLD, f"plan_plain_{name}.npz")
    pre = os.path.join(GOLD, f"plan_prepost_{name}.npz")
    P = len(np.load(plain)["begin"]) - 1
    port = 29800 + (os.getpid() % 150) + ord(name)
    mp.spawn(_plan_worker, args=(P, port, plain, pre, str(tmp_path)), nprocs=P, join=True)
    for r in range(P):
        msg = open(os.path.join(str(tmp_path), f"r{r}.txt")).read()
        assert msg == "", f"rank {r}: {msg}"
