"""Golden vectors of the reference's OWN Aggregator / Communicator / DistSAGE, run here on CPU.

    python tests/golden/make_aggregator_golden.py <reference_root>
    python tests/golden/make_aggregator_golden.py gcn <reference_root>   # train_gcn_config1.npz (minutes)

What runs: the unmodified Python of the reference (model/layers/aggregator.py, communicator.py,
quantizer.py, data_manager/*, model/ops/spmm_kernel.py, model/DistSAGE.py, model/layers/sageconv.py)
as P gloo processes, over its compiled native module (oracle/_ref) for spmm and the x86 quantisers.

What had to be stood in for, and how (tests-only, none of it arithmetic of the path except the
last item):
  * torch_sparse.SparseTensor / torch_scatter.segment_csr / torch_geometric.* -- forks that are
    not in the reference's repository: minimal holders defined below (canonical CSR/CSC sorting,
    the four work-range accessors, a segment sum, nn.Module / nn.Linear aliases);
  * Communicator.init_dist_group -- hard-codes MPI / oneCCL: the process group is gloo;
  * dist.all_to_all (list form, DataProcessor.py:77,94) -- unsupported by gloo: expressed with
    all_to_all_single, same payload;
  * computation_ops.{quantize,dequantize}_tensor_for_all_procs -- ARM SVE only
    (quantization_arm.cpp:364-479): the C restatement in oracle/gnnagg_oracle.c.  The int2 vectors
    are therefore "reference Python + restated ARM kernel"; everything else is reference code.

Outputs: tests/golden/aggr_<case>.npz (inputs, per-rank forward output, input gradient, halo buffers,
codes) and tests/golden/train_sage.npz (20-epoch loss curve of the reference's DistSAGE).
"""
import contextlib
import io
import os
import sys
import types

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

HERE = os.path.dirname(os.path.abspath(__file__))
REPO = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, REPO)


# ------------------------------------------------------------------------------------------------
class _Storage:
    def __init__(self, o):
        self.o = o

    def colptr(self):
        return self.o._csc()[0]

    def row_T(self):
        return self.o._csc()[1]

    def value_T(self):
        return self.o._csc()[2]


class ShimSparseTensor:
    """Holder with the surface model/ops/spmm_kernel.py uses.  Canonical order: row-major, then
    column ascending (stable, duplicates kept); CSC: column-major, rows ascending."""

    def __init__(self, row=None, col=None, value=None, sparse_sizes=None, **kw):
        M, K = sparse_sizes
        key = row.to(torch.int64) * max(K, 1) + col.to(torch.int64)
        perm = torch.sort(key, stable=True)[1]
        self.row, self.col, self.value = row[perm].to(torch.int64), col[perm].to(torch.int64), value[perm]
        self.sizes = (int(M), int(K))
        self.rowptr = torch.zeros(M + 1, dtype=torch.int64)
        torch.cumsum(torch.bincount(self.row, minlength=M), 0, out=self.rowptr[1:])
        self._t = None
        self._wr = (torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32))
        self._wrt = (torch.empty(0, dtype=torch.int32), torch.empty(0, dtype=torch.int32))
        self.storage = _Storage(self)

    def csr(self):
        return self.rowptr, self.col, self.value

    def sparse_size(self, i):
        return self.sizes[i]

    def _csc(self):
        if self._t is None:
            perm = torch.sort(self.col, stable=True)[1]
            colptr = torch.zeros(self.sizes[1] + 1, dtype=torch.int64)
            torch.cumsum(torch.bincount(self.col, minlength=self.sizes[1]), 0, out=colptr[1:])
            self._t = (colptr, self.row[perm].contiguous(), self.value[perm].contiguous())
        return self._t

    def get_work_range(self):
        return self._wr

    def set_work_range(self, r, c):
        self._wr = (r, c)

    def get_work_range_for_transpose(self):
        return self._wrt

    def set_work_range_for_transpose(self, r, c):
        self._wrt = (r, c)


def install_shims(ref_root):
    import oracle

    a64 = os.path.join(ref_root, "self_benchmark", "a64fx")
    ts = types.ModuleType("torch_sparse")
    ts.SparseTensor = ShimSparseTensor
    # names imported (never called) by the dead legacy layer model/layers/sageconv_forpre.py:6-7
    ts.fill_diag = None
    ts.sum = None
    sys.modules["torch_sparse"] = ts

    tsc = types.ModuleType("torch_scatter")

    def segment_csr(value, rowptr, out=None, reduce="sum"):
        c = torch.zeros(value.numel() + 1, dtype=torch.float64)
        torch.cumsum(value.double(), 0, out=c[1:])
        return (c[rowptr[1:]] - c[rowptr[:-1]]).to(value.dtype)

    tsc.segment_csr = segment_csr
    sys.modules["torch_scatter"] = tsc

    ref = oracle.load_reference_module()
    if ref is None:
        raise SystemExit("build oracle/_ref first: python oracle/build_ref.py")
    ops = types.ModuleType("computation_ops")
    for n in ("spmm", "quantize_tensor_v1", "dequantize_tensor_v1"):
        setattr(ops, n, getattr(ref, n))

    def quantize_tensor_for_all_procs(inp, out, params, work_range, num_procs, bits):
        codes, p = oracle.quantize_int2_for_all_procs(inp.numpy(), work_range.numpy())
        out.view(-1)[: codes.size].copy_(torch.from_numpy(codes).view(-1))
        params.copy_(torch.from_numpy(p))

    def dequantize_tensor_for_all_procs(inp, out, params, work_range, num_procs, bits):
        F = out.size(1)
        y = oracle.dequantize_int2_for_all_procs(inp.numpy().reshape(-1, F), work_range.numpy(), params.numpy())
        out.copy_(torch.from_numpy(y))

    ops.quantize_tensor_for_all_procs = quantize_tensor_for_all_procs
    ops.dequantize_tensor_for_all_procs = dequantize_tensor_for_all_procs
    ops.quantize_tensor = ref.quantize_tensor
    ops.dequantize_tensor = ref.dequantize_tensor
    sys.modules["computation_ops"] = ops

    sys.path.insert(0, a64)
    sys.path.insert(0, os.path.join(a64, "model", "ops"))
    tg = types.ModuleType("torch_geometric")
    tgnn = types.ModuleType("torch_geometric.nn")
    import importlib.util

    spec = importlib.util.spec_from_file_location("torch_geometric.nn.spmm_kernel",
                                                  os.path.join(a64, "model", "ops", "spmm_kernel.py"))
    sk = importlib.util.module_from_spec(spec)
    sys.modules["torch_geometric.nn.spmm_kernel"] = sk
    spec.loader.exec_module(sk)
    tgnn.spmm_kernel = sk
    conv = types.ModuleType("torch_geometric.nn.conv")

    class MessagePassing(torch.nn.Module):
        def __init__(self, aggr="add", **kw):
            super().__init__()

    conv.MessagePassing = MessagePassing
    dense = types.ModuleType("torch_geometric.nn.dense")
    lin = types.ModuleType("torch_geometric.nn.dense.linear")
    lin.Linear = torch.nn.Linear
    inits = types.ModuleType("torch_geometric.nn.inits")
    inits.zeros = None
    tgnn.inits = inits
    for name, m in (("torch_geometric", tg), ("torch_geometric.nn", tgnn), ("torch_geometric.nn.conv", conv),
                    ("torch_geometric.nn.dense", dense), ("torch_geometric.nn.dense.linear", lin),
                    ("torch_geometric.nn.inits", inits)):
        sys.modules[name] = m
    tg.nn = tgnn
    tgnn.conv = conv
    tgnn.dense = dense
    dense.linear = lin

    # list-form all_to_all on gloo
    def all_to_all_list(out_list, in_list, group=None, async_op=False):
        inp = torch.cat([t.reshape(-1) for t in in_list])
        out = torch.empty(sum(t.numel() for t in out_list), dtype=inp.dtype)
        dist.all_to_all_single(out, inp, [t.numel() for t in out_list], [t.numel() for t in in_list])
        off = 0
        for t in out_list:
            t.copy_(out[off: off + t.numel()].view_as(t))
            off += t.numel()

    dist.all_to_all = all_to_all_list


def make_graph(seed, P, n_per, deg):
    rng = np.random.default_rng(seed)
    sizes = rng.integers(max(1, n_per // 2), n_per + 1, size=P)
    begin = np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64)
    N = int(begin[-1])
    E = N * deg
    src = rng.integers(0, N, size=E)
    dst = rng.integers(0, N, size=E)
    hubs = rng.integers(0, N, size=max(2, N // 40))
    src[: E // 5] = rng.choice(hubs, size=E // 5)
    dst[E // 5: 2 * E // 5] = rng.choice(hubs, size=2 * E // 5 - E // 5)
    src = np.concatenate([src, src[: E // 20]])
    dst = np.concatenate([dst, dst[: E // 20]])
    return begin, src.astype(np.int64), dst.astype(np.int64)


def partition(src, dst, begin, r):
    m = (dst >= begin[r]) & (dst < begin[r + 1])
    s, d = src[m], dst[m]
    loc = (s >= begin[r]) & (s < begin[r + 1])
    local = np.stack([s[loc] - begin[r], d[loc] - begin[r]]).astype(np.int64)
    remote = np.stack([s[~loc], d[~loc] - begin[r]]).astype(np.int64)
    return local, remote


def build_reference_graph(local, remote, begin, rank, P, max_feat, bits, is_pre):
    from data_manager.DataLoader import get_distributed_graph, get_distributed_graph_for_pre_aggressive

    le = [torch.from_numpy(local[0].copy()), torch.from_numpy(local[1].copy())]
    re = [torch.from_numpy(remote[0].copy()), torch.from_numpy(remote[1].copy())]
    bt = torch.from_numpy(begin)
    n = int(begin[rank + 1] - begin[rank])
    if is_pre:
        return get_distributed_graph_for_pre_aggressive(le, re, bt, n, max_feat, rank, P, bits)
    nodes = torch.arange(int(begin[rank]), int(begin[rank + 1]), dtype=torch.int64).view(-1, 1).repeat(1, 2)
    return get_distributed_graph(le, re, nodes, bt, n, max_feat, P, bits)


def aggr_worker(rank, P, port, case, ref_root, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.set_num_threads(2)
    install_shims(ref_root)
    from communicator import Communicator
    from quantizer import Quantizer_for_all_procs
    from time_recorder import TimeRecorder
    from model.layers.aggregator import Aggregator

    name, seed, n_per, deg, F, bits, is_pre = case
    c = Communicator(bits, is_async=True)
    c.rank, c.world_size = rank, P
    Quantizer_for_all_procs(P, bits)
    TimeRecorder(2, 2)
    begin, src, dst = make_graph(seed, P, n_per, deg)
    N = int(begin[-1])
    rng = np.random.default_rng(seed + 1)
    X = rng.standard_normal((N, F)).astype(np.float32)
    G = rng.standard_normal((N, F)).astype(np.float32)
    local, remote = partition(src, dst, begin, rank)
    with contextlib.redirect_stdout(io.StringIO()):
        graph = build_reference_graph(local, remote, begin, rank, P, F, bits, is_pre)
        b0, b1 = int(begin[rank]), int(begin[rank + 1])
        x = torch.from_numpy(X[b0:b1].copy()).requires_grad_()
        out = Aggregator.apply(graph, x, 0, bits, is_pre, True)
        fwd_recv = graph.comm_buf.recv_buf.clone()
        fwd_send = graph.comm_buf.send_buf.clone()
        extra = {}
        if bits == 2:
            q = graph.comm_buf_for_quantization
            extra["fwd_codes"] = q.quantized_send_data_buf.clone().numpy()
            extra["fwd_params"] = q.quantized_send_params_buf_fp32.clone().numpy()
        out.backward(torch.from_numpy(G[b0:b1].copy()))
    o = dict(out=out.detach().numpy(), grad=x.grad.numpy(), fwd_recv=fwd_recv.numpy(), fwd_send=fwd_send.numpy(),
             recv_splits=np.array(graph.comm_splits.recv_splits), send_splits=np.array(graph.comm_splits.send_splits),
             in_degrees=graph.in_degrees.numpy(), **extra)
    np.savez_compressed(os.path.join(out_dir, f"_tmp_{name}_r{rank}.npz"), **o)
    dist.barrier()
    if rank == 0:
        merged = dict(begin=begin, src=src, dst=dst, X=X, G=G, F=np.array(F), bits=np.array(bits),
                      is_pre=np.array(int(is_pre)), P=np.array(P))
        for r in range(P):
            p = os.path.join(out_dir, f"_tmp_{name}_r{r}.npz")
            with np.load(p) as z:
                for k in z.files:
                    merged[f"r{r}_{k}"] = z[k]
            os.unlink(p)
        np.savez_compressed(os.path.join(out_dir, f"aggr_{name}.npz"), **merged)
    dist.destroy_process_group()


def train_worker(rank, P, port, cfg, ref_root, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.set_num_threads(2)
    install_shims(ref_root)
    import torch.nn.functional as Fn
    from assigner import Assigner
    from communicator import Communicator
    from quantizer import Quantizer_for_all_procs
    from time_recorder import TimeRecorder
    from model import create_model_and_optimizer, set_random_seed

    bits, is_pre = cfg["num_bits"], cfg["is_pre_delay"]
    c = Communicator(bits, is_async=True)
    c.rank, c.world_size = rank, P
    Quantizer_for_all_procs(P, bits)
    begin, src, dst = make_graph(cfg["graph_seed"], P, cfg["n_per"], cfg["deg"])
    N = int(begin[-1])
    rng = np.random.default_rng(cfg["graph_seed"] + 1)
    X = rng.standard_normal((N, cfg["in_channels"])).astype(np.float32)
    labels = rng.integers(0, cfg["out_channels"], size=N).astype(np.int64)
    train_mask = rng.random(N) < 0.5
    local, remote = partition(src, dst, begin, rank)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    losses = []
    with contextlib.redirect_stdout(io.StringIO()):
        set_random_seed(cfg["random_seed"])
        model, optimizer = create_model_and_optimizer(cfg)
        init_state = {k: v.detach().clone().numpy() for k, v in model.state_dict().items()}
        max_feat = max(cfg["in_channels"], cfg["hidden_channels"], cfg["out_channels"])
        graph = build_reference_graph(local, remote, begin, rank, P, max_feat, bits, is_pre)
        Assigner(bits, cfg["num_layers"], torch.tensor([1.0, 1.0, 1.0]), 1, graph.comm_buf.send_buf.size(0),
                 graph.comm_buf.recv_buf.size(0))
        TimeRecorder(cfg["num_layers"], cfg["num_epochs"])
        x = torch.from_numpy(X[b0:b1].copy())
        y = torch.from_numpy(labels[b0:b1].copy())
        tm = torch.from_numpy(np.nonzero(train_mask[b0:b1])[0])
        for epoch in range(cfg["num_epochs"]):
            model.train()
            optimizer.zero_grad()
            out = model(graph, x)
            loss = Fn.nll_loss(out[tm], y[tm])
            loss.backward()
            optimizer.step()
            losses.append(float(loss))
            TimeRecorder.ctx.next_epoch()
    np.savez_compressed(os.path.join(out_dir, f"_tmp_train_r{rank}.npz"), losses=np.array(losses, dtype=np.float64),
                        **{"w_" + k.replace("module.", ""): v for k, v in init_state.items()})
    dist.barrier()
    if rank == 0:
        merged = dict(begin=begin, src=src, dst=dst, X=X, labels=labels, train_mask=train_mask,
                      cfg_keys=np.array(sorted(k for k in cfg if not isinstance(cfg[k], str))),
                      cfg_vals=np.array([float(cfg[k]) for k in sorted(k for k in cfg if not isinstance(cfg[k], str))]))
        for r in range(P):
            p = os.path.join(out_dir, f"_tmp_train_r{r}.npz")
            with np.load(p) as z:
                for k in z.files:
                    if k == "losses":
                        merged[f"r{r}_losses"] = z[k]
                    elif r == 0:
                        merged[k] = z[k]
            os.unlink(p)
        np.savez_compressed(os.path.join(out_dir, f"train_{cfg['name']}.npz"), **merged)
    dist.destroy_process_group()


def gcn_config1_worker(rank, P, port, cfg, ref_root, out_dir):
    """BASELINE configuration 1 at full size: 2-layer GCN, Erdos-Renyi 131 072 nodes, average degree 16,
    self-loops, symmetric normalisation, 2 contiguous blocks, F 128 -> 128 -> 16, Adam lr 0.01, fp32
    halo, 20 epochs.  The reference has no GCN layer; the layer below wraps the REFERENCE's Aggregator
    exactly as gnn_benchmark_b200.model.DistGCNConv wraps the CUDA one (row scaling by d^-1/2 before and
    after the aggregation; transform first when in > out)."""
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=P)
    torch.set_num_threads(4)
    install_shims(ref_root)
    import torch.nn.functional as Fn
    from communicator import Communicator
    from quantizer import Quantizer_for_all_procs
    from time_recorder import TimeRecorder
    from model.layers.aggregator import Aggregator
    from gnn_benchmark_b200 import graphgen

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
            h = Aggregator.apply(graph, h * dinv, layer, 32, False, self.training)
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

    c = Communicator(32, is_async=True)
    c.rank, c.world_size = rank, P
    Quantizer_for_all_procs(P, 32)
    n = cfg["nodes"]
    src, dst = graphgen.erdos_renyi_edges(n, n * cfg["avg_degree"] // 2, seed=cfg["graph_seed"], device="cpu")
    src, dst = graphgen.symmetrize(src, dst, n, self_loops=True)
    begin = graphgen.contiguous_partitions(n, P)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    g = torch.Generator().manual_seed(cfg["graph_seed"] + 1)
    X = torch.randn(n, cfg["dims"][0], generator=g)
    labels = torch.randint(0, cfg["dims"][-1], (n,), generator=g)
    train_mask = torch.rand(n, generator=g) < 0.5
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    losses = []
    with contextlib.redirect_stdout(io.StringIO()):
        torch.manual_seed(cfg["random_seed"])
        model = RefGCN(cfg["dims"])
        for conv in model.convs:
            conv.reset_parameters()
        ddp = torch.nn.parallel.DistributedDataParallel(model)
        opt = torch.optim.Adam(ddp.parameters(), lr=0.01)
        graph = build_reference_graph(local.numpy(), remote.numpy(), begin.numpy(), rank, P, max(cfg["dims"]), 32, False)
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
    np.save(os.path.join(out_dir, f"_tmp_gcn_r{rank}.npy"), np.array(losses, dtype=np.float64))
    dist.barrier()
    if rank == 0:
        merged = {k: np.array(v) for k, v in cfg.items() if k != "name"}
        for r in range(P):
            pth = os.path.join(out_dir, f"_tmp_gcn_r{r}.npy")
            merged[f"r{r}_losses"] = np.load(pth)
            os.unlink(pth)
        np.savez_compressed(os.path.join(out_dir, "train_gcn_config1.npz"), **merged)
    dist.destroy_process_group()


GCN_CONFIG1 = dict(name="gcn_config1", nodes=131072, avg_degree=16, dims=[128, 128, 16], num_epochs=20, random_seed=4321,
                   graph_seed=20261126)

AGGR_CASES = [
    # name, seed, n_per, deg, F, bits, is_pre
    ("plain_fp32_p2", 11, 150, 5, 128, 32, False),
    ("plain_fp32_p3_f32", 12, 120, 4, 32, 32, False),
    ("pre_fp32_p3", 13, 100, 5, 128, 32, True),
    ("plain_int2_p2", 14, 150, 5, 128, 2, False),
    ("pre_int2_p3", 15, 70, 4, 256, 2, True),
    ("plain_int2_p4_f100", 16, 70, 4, 100, 2, False),
]
AGGR_P = {"plain_fp32_p2": 2, "plain_fp32_p3_f32": 3, "pre_fp32_p3": 3, "plain_int2_p2": 2, "pre_int2_p3": 3,
          "plain_int2_p4_f100": 4}

TRAIN_CFGS = [
    dict(name="sage_fp32_p2", P=2, model_name="sage", in_channels=64, hidden_channels=128, out_channels=16,
         num_layers=3, dropout=0.0, lr=0.01, weight_decay=0.0, num_epochs=20, random_seed=1234, num_bits=32,
         is_pre_delay=False, graph_seed=21, n_per=400, deg=6),
    dict(name="sage_int2_pre_p2", P=2, model_name="sage", in_channels=64, hidden_channels=128, out_channels=16,
         num_layers=3, dropout=0.0, lr=0.01, weight_decay=0.0, num_epochs=20, random_seed=1234, num_bits=2,
         is_pre_delay=True, graph_seed=22, n_per=400, deg=6),
]


def main():
    if len(sys.argv) < 2:
        sys.exit("usage: make_aggregator_golden.py <reference_root> | gcn <reference_root>")
    ref_root = sys.argv[1]
    port = 29610
    for case in AGGR_CASES:
        P = AGGR_P[case[0]]
        mp.spawn(aggr_worker, args=(P, port, case, ref_root, HERE), nprocs=P, join=True)
        port += 1
        print("wrote aggr_%s.npz" % case[0])
    for cfg in TRAIN_CFGS:
        mp.spawn(train_worker, args=(cfg["P"], port, cfg, ref_root, HERE), nprocs=cfg["P"], join=True)
        port += 1
        print("wrote train_%s.npz" % cfg["name"])


def main_gcn():
    if len(sys.argv) < 3:
        sys.exit("usage: make_aggregator_golden.py gcn <reference_root>")
    ref_root = sys.argv[2]
    mp.spawn(gcn_config1_worker, args=(2, 29690, GCN_CONFIG1, ref_root, HERE), nprocs=2, join=True)
    print("wrote train_gcn_config1.npz")


if __name__ == "__main__":
    if len(sys.argv) > 1 and sys.argv[1] == "gcn":
        main_gcn()
    else:
        main()
