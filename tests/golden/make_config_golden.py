"""Golden vectors at the model dimensions of BASELINE configurations 4 and 5, and a teacher-forcing
fixture for the 2-bit halo, all from the reference's OWN Aggregator / Communicator / plan builders
(and its DistSAGE) run here on CPU as gloo ranks.

    python tests/golden/make_config_golden.py <reference_root> [gcn5] [sage4] [teacher]

gcn5    train_gcn_config5_scaled.npz  -- 3-layer GCN 128 -> 256 -> 256 -> 172, 8 ranks, 2-bit halo,
        seeded Chung-Lu (exponent 2.1) graph of 2^15 vertices with the configuration's mean degree,
        randomly relabelled, 1 % train mask, Adam lr 0.01, 20 epochs: per-rank loss curves.  The
        reference has no GCN layer: the same wrapper as for configuration 1 (row scaling by d^-1/2
        either side of the REFERENCE's Aggregator; transform first when in > out).
sage4   train_sage_config4_scaled_{fp32,int2}.npz -- the reference's DistSAGE 100 -> 256 -> 256 -> 47,
        4 ranks, Chung-Lu graph of 2^14 vertices with the configuration's mean degree, 8 % train
        mask: per-rank loss curves with the fp32 and the 2-bit halo.
teacher teacher_sage_int2_p4.npz -- the reference's DistSAGE with the 2-bit halo on a small 4-rank
        graph; at three epochs every Aggregator call is recorded: its input, its output, the
        incoming and outgoing gradients, and the codes and parameters it put on the wire in both
        directions.  Feeding the recorded inputs to another implementation must give the same codes
        bit for bit: that separates "the kernels differ" from "a one-ulp difference upstream moved a
        value across a 2-bit rounding boundary".

Graphs and features are regenerated from their seeds by the tests (the generators are pure torch
and run on the CPU); only seeds, sizes and results are stored.  The stand-ins for the packages the
reference imports but does not contain are those of make_aggregator_golden.py.
"""
import contextlib
import io
import os
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))

from make_aggregator_golden import build_reference_graph, install_shims, make_graph, partition  # noqa: E402
from util import synthetic_problem  # noqa: E402  (tests/util.py: the tests rebuild the same inputs with it)


def _save_losses(cfg, rank, P, losses, out_dir):
    tmp = os.path.join(out_dir, f"_tmp_{cfg['name']}_r{rank}.npy")
    np.save(tmp, np.array(losses, dtype=np.float64))
    dist.barrier()
    if rank == 0:
        merged = {k: np.array(v) for k, v in cfg.items() if k != "name"}
        for r in range(P):
            pth = os.path.join(out_dir, f"_tmp_{cfg['name']}_r{r}.npy")
            merged[f"r{r}_losses"] = np.load(pth)
            os.unlink(pth)
        np.savez_compressed(os.path.join(out_dir, f"train_{cfg['name']}.npz"), **merged)


def _init(rank, P, port, ref_root, bits, threads):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.set_num_threads(threads)
    install_shims(ref_root)
    from communicator import Communicator
    from quantizer import Quantizer_for_all_procs

    c = Communicator(bits, is_async=True)
    c.rank, c.world_size = rank, P
    Quantizer_for_all_procs(P, bits)


def gcn_worker(rank, P, port, cfg, ref_root, out_dir):
    _init(rank, P, port, ref_root, cfg["num_bits"], 1)
    import torch.nn.functional as Fn
    from model.layers.aggregator import Aggregator
    from time_recorder import TimeRecorder

    bits = cfg["num_bits"]

    class RefGCNConv(torch.nn.Module):
        def __init__(self, cin, cout):
            super().__init__()
            self.cin, self.cout = cin, cout
            self.lin = torch.nn.Linear(cin, cout, bias=False)
            self.bias = torch.nn.Parameter(torch.zeros(cout))

        def reset_parameters(self):
            torch.nn.init.xavier_uniform_(self.lin.weight)
            torch.nn.init.zeros_(self.bias)

        def forward(self, graph, x, layer):
            dinv = graph.in_degrees.rsqrt()
            first = self.cin > self.cout
            h = self.lin(x) if first else x
            h = Aggregator.apply(graph, h * dinv, layer, bits, False, self.training)
            h = h * dinv
            if not first:
                h = self.lin(h)
            return h + self.bias

    class RefGCN(torch.nn.Module):
        def __init__(self, dims):
            super().__init__()
            self.convs = torch.nn.ModuleList(RefGCNConv(dims[i], dims[i + 1]) for i in range(len(dims) - 1))

        def forward(self, graph, x):
            for i, conv in enumerate(self.convs[:-1]):
                x = Fn.relu(conv(graph, x, i))
            return Fn.log_softmax(self.convs[-1](graph, x, len(self.convs) - 1), dim=1)

    from gnn_benchmark_b200 import graphgen

    src, dst, begin, X, labels, train_mask = synthetic_problem(cfg)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    losses = []
    with contextlib.redirect_stdout(io.StringIO()):
        torch.manual_seed(cfg["random_seed"])
        model = RefGCN(cfg["dims"])
        for conv in model.convs:
            conv.reset_parameters()
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        opt = torch.optim.Adam(ddp.parameters(), lr=0.01)
        graph = build_reference_graph(local.numpy(), remote.numpy(), begin.numpy(), rank, P, max(cfg["dims"]), bits,
                                      False)
        TimeRecorder(len(cfg["dims"]) - 1, cfg["num_epochs"])
        x, y = X[b0:b1].clone(), labels[b0:b1].clone()
        tm = torch.nonzero(train_mask[b0:b1]).view(-1)
        for epoch in range(cfg["num_epochs"]):
            ddp.train()
            opt.zero_grad()
            out = ddp(graph, x)
            loss = Fn.nll_loss(out[tm], y[tm])
            loss.backward()
            opt.step()
            losses.append(float(loss.detach()))
            TimeRecorder.ctx.next_epoch()
    _save_losses(cfg, rank, P, losses, out_dir)
    dist.destroy_process_group()


def _sage_cfg(cfg):
    d = cfg["dims"]
    return dict(model_name="sage", in_channels=d[0], hidden_channels=d[1], out_channels=d[-1], num_layers=len(d) - 1,
                dropout=0.0, lr=0.01, weight_decay=0.0, num_epochs=cfg["num_epochs"], num_bits=cfg["num_bits"],
                is_pre_delay=bool(cfg["is_pre_delay"]))


def sage_worker(rank, P, port, cfg, ref_root, out_dir):
    """The reference's own DistSAGE (model/DistSAGE.py, model/layers/sageconv.py) and epoch loop."""
    _init(rank, P, port, ref_root, cfg["num_bits"], 2)
    import torch.nn.functional as Fn
    from assigner import Assigner
    from model import create_model_and_optimizer, set_random_seed
    from time_recorder import TimeRecorder
    from gnn_benchmark_b200 import graphgen

    src, dst, begin, X, labels, train_mask = synthetic_problem(cfg)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    mcfg = _sage_cfg(cfg)
    losses = []
    with contextlib.redirect_stdout(io.StringIO()):
        set_random_seed(cfg["random_seed"])
        model, optimizer = create_model_and_optimizer(mcfg)
        graph = build_reference_graph(local.numpy(), remote.numpy(), begin.numpy(), rank, P, max(cfg["dims"]),
                                      cfg["num_bits"], bool(cfg["is_pre_delay"]))
        Assigner(cfg["num_bits"], mcfg["num_layers"], torch.tensor([1.0, 1.0, 1.0]), 1, graph.comm_buf.send_buf.size(0),
                 graph.comm_buf.recv_buf.size(0))
        TimeRecorder(mcfg["num_layers"], cfg["num_epochs"])
        x, y = X[b0:b1].clone(), labels[b0:b1].clone()
        tm = torch.nonzero(train_mask[b0:b1]).view(-1)
        for epoch in range(cfg["num_epochs"]):
            model.train()
            optimizer.zero_grad()
            out = model(graph, x)
            loss = Fn.nll_loss(out[tm], y[tm])
            loss.backward()
            optimizer.step()
            losses.append(float(loss.detach()))
            TimeRecorder.ctx.next_epoch()
    _save_losses(cfg, rank, P, losses, out_dir)
    dist.destroy_process_group()


def teacher_worker(rank, P, port, cfg, ref_root, out_dir):
    """DistSAGE with the 2-bit halo; every Aggregator call of the epochs in cfg["record_epochs"] is
    recorded through a subclass that only observes (the arithmetic is the reference's)."""
    _init(rank, P, port, ref_root, cfg["num_bits"], 2)
    import torch.nn.functional as Fn
    from assigner import Assigner
    from model import create_model_and_optimizer, set_random_seed
    from model.layers import sageconv
    from model.layers.aggregator import Aggregator
    from time_recorder import TimeRecorder

    rec = {}
    state = {"epoch": -1}

    def on(epoch):
        return epoch in cfg["record_epochs"]

    class Observed(Aggregator):
        @staticmethod
        def forward(ctx, graph, x, layer, num_bits, is_pre_delay, is_training):
            out = Aggregator.forward(ctx, graph, x, layer, num_bits, is_pre_delay, is_training)
            if on(state["epoch"]):
                q = graph.comm_buf_for_quantization
                k = f"e{state['epoch']}_l{layer}"
                rec[k + "_x"] = x.detach().clone().numpy()
                rec[k + "_out"] = out.detach().clone().numpy()
                rec[k + "_fwd_codes"] = q.quantized_send_data_buf.clone().numpy()
                rec[k + "_fwd_params"] = q.quantized_send_params_buf_fp32.clone().numpy()
            return out

        @staticmethod
        def backward(ctx, g):
            res = Aggregator.backward(ctx, g)
            if on(state["epoch"]):
                q = ctx.graph.comm_buf_for_quantization
                k = f"e{state['epoch']}_l{ctx.layer}"
                rec[k + "_g"] = g.detach().clone().numpy()
                rec[k + "_grad"] = res[1].detach().clone().numpy()
                # backward: the receive-side buffers are the ones sent (the roles swap)
                rec[k + "_bwd_codes"] = q.quantized_recv_data_buf.clone().numpy()
                rec[k + "_bwd_params"] = q.quantized_recv_params_buf_fp32.clone().numpy()
            return res

    sageconv.Aggregator = Observed
    begin, src, dst = make_graph(cfg["graph_seed"], P, cfg["n_per"], cfg["deg"])
    N = int(begin[-1])
    rng = np.random.default_rng(cfg["graph_seed"] + 1)
    d = cfg["dims"]
    X = rng.standard_normal((N, d[0])).astype(np.float32)
    labels = rng.integers(0, d[-1], size=N).astype(np.int64)
    train_mask = rng.random(N) < 0.5
    local, remote = partition(src, dst, begin, rank)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    mcfg = _sage_cfg(cfg)
    losses = []
    with contextlib.redirect_stdout(io.StringIO()):
        set_random_seed(cfg["random_seed"])
        model, optimizer = create_model_and_optimizer(mcfg)
        graph = build_reference_graph(local, remote, begin, rank, P, max(d), cfg["num_bits"], bool(cfg["is_pre_delay"]))
        Assigner(cfg["num_bits"], mcfg["num_layers"], torch.tensor([1.0, 1.0, 1.0]), 1, graph.comm_buf.send_buf.size(0),
                 graph.comm_buf.recv_buf.size(0))
        TimeRecorder(mcfg["num_layers"], cfg["num_epochs"])
        x = torch.from_numpy(X[b0:b1].copy())
        y = torch.from_numpy(labels[b0:b1].copy())
        tm = torch.from_numpy(np.nonzero(train_mask[b0:b1])[0])
        for epoch in range(cfg["num_epochs"]):
            state["epoch"] = epoch
            model.train()
            optimizer.zero_grad()
            out = model(graph, x)
            loss = Fn.nll_loss(out[tm], y[tm])
            loss.backward()
            optimizer.step()
            losses.append(float(loss.detach()))
            TimeRecorder.ctx.next_epoch()
    np.savez_compressed(os.path.join(out_dir, f"_tmp_teacher_r{rank}.npz"), losses=np.array(losses), **rec)
    dist.barrier()
    if rank == 0:
        merged = dict(begin=begin, src=src, dst=dst, P=np.array(P), dims=np.array(d), num_bits=np.array(cfg["num_bits"]),
                      is_pre_delay=np.array(int(cfg["is_pre_delay"])), record_epochs=np.array(cfg["record_epochs"]))
        for r in range(P):
            pth = os.path.join(out_dir, f"_tmp_teacher_r{r}.npz")
            with np.load(pth) as z:
                for k in z.files:
                    merged[f"r{r}_{k}"] = z[k]
            os.unlink(pth)
        np.savez_compressed(os.path.join(out_dir, f"teacher_{cfg['name']}.npz"), **merged)
    dist.destroy_process_group()


# mean degrees of the configurations: 5 -> 1.6 B directed edges / 111 M vertices = 14.4 drawn per vertex;
# 4 -> 61.9 M undirected edges / 2.45 M vertices = 25.3 drawn per vertex
GCN5 = dict(name="gcn_config5_scaled", P=8, nodes=1 << 15, edges=int(14.4 * (1 << 15)), self_loops=1, dims=[128, 256, 256, 172],
            num_bits=2, is_pre_delay=0, train_frac=0.01, num_epochs=20, random_seed=4322, graph_seed=20261130)
SAGE4 = [
    dict(name="sage_config4_scaled_fp32", P=4, nodes=1 << 14, edges=int(25.3 * (1 << 14)), self_loops=0, dims=[100, 256, 256, 47],
         num_bits=32, is_pre_delay=0, train_frac=0.08, num_epochs=20, random_seed=4323, graph_seed=20261129),
    dict(name="sage_config4_scaled_int2", P=4, nodes=1 << 14, edges=int(25.3 * (1 << 14)), self_loops=0, dims=[100, 256, 256, 47],
         num_bits=2, is_pre_delay=0, train_frac=0.08, num_epochs=20, random_seed=4323, graph_seed=20261129),
]
TEACHER = dict(name="sage_int2_p4", P=4, n_per=96, deg=5, dims=[64, 128, 128, 16], num_bits=2, is_pre_delay=0,
               num_epochs=20, random_seed=1235, graph_seed=23, record_epochs=[0, 9, 19])


def main():
    args = [a for a in sys.argv[1:]]
    ref_root = args[0] if args and os.path.isdir(args[0]) else os.environ.get("GNNAGG_REFERENCE_ROOT")
    if not ref_root:
        raise SystemExit("usage: python tests/golden/make_config_golden.py <reference_root> [gcn5] [sage4] [teacher]")
    what = set(a for a in args if a in ("gcn5", "sage4", "teacher")) or {"gcn5", "sage4", "teacher"}
    port = 29810
    if "teacher" in what:
        mp.spawn(teacher_worker, args=(TEACHER["P"], port, TEACHER, ref_root, HERE), nprocs=TEACHER["P"], join=True)
        print("wrote teacher_%s.npz" % TEACHER["name"])
    if "sage4" in what:
        for cfg in SAGE4:
            port += 1
            mp.spawn(sage_worker, args=(cfg["P"], port, cfg, ref_root, HERE), nprocs=cfg["P"], join=True)
            print("wrote train_%s.npz" % cfg["name"])
    if "gcn5" in what:
        port += 1
        mp.spawn(gcn_worker, args=(GCN5["P"], port, GCN5, ref_root, HERE), nprocs=GCN5["P"], join=True)
        print("wrote train_%s.npz" % GCN5["name"])


if __name__ == "__main__":
    main()
