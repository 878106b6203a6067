"""Full-batch epoch time of a GNN over the aggregation path, on synthetic power-law graphs.

    torchrun --nproc-per-node N bench_epoch.py --model gcn --nodes 111000000 \\
        --edges 1600000000 --in-channels 128 --hidden 256 --out-channels 172 --layers 3 --bits 2

Shapes: `--model sage --nodes 2450000 --edges 61900000 --in-channels 100 --hidden 256 --out-channels 47
--train-frac 0.08` is the products-shaped configuration, the default the papers100M-shaped one
(scale both down with --nodes/--edges to fit fewer GPUs).  The graph is a seeded Chung-Lu power-law
graph (exponent 2.1), symmetrised, with self-loops, randomly relabelled and cut into N contiguous
vertex blocks; every rank generates its own block.  The epoch's timed region is forward start ->
optimiser step end (the reference's `Time:` field, train.py:84-98); epoch 0 is excluded from the mean
(the reference's scraper does the same).  Prints one JSON line on rank 0: epoch time, aggregated
edges/s (edges x aggregation passes actually executed per step), halo volume.
"""
import argparse
import json
import time

import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from gnn_benchmark_b200 import dense, graphgen  # noqa: E402
from gnn_benchmark_b200.communicator import Communicator  # noqa: E402
from gnn_benchmark_b200.data_manager.DataLoader import build_graph  # noqa: E402
from gnn_benchmark_b200.model import create_model_and_optimizer, set_random_seed  # noqa: E402
from gnn_benchmark_b200.quantizer import Quantizer_for_all_procs  # noqa: E402
from gnn_benchmark_b200.time_recorder import TimeRecorder  # noqa: E402
from gnn_benchmark_b200.train import train  # noqa: E402


def aggregation_passes(model_name: str, dims) -> int:
    """Aggregations per training step: one forward per layer, one backward per layer whose aggregated
    tensor needs a gradient (not layer 0 when it aggregates the raw features)."""
    L = len(dims) - 1
    if model_name == "sage":
        return L + (L - 1)
    back = sum(1 for i in range(L) if i > 0 or dims[i] > dims[i + 1])  # gcn: transform-first layers carry grad
    return L + back


def make_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="gcn", choices=["gcn", "sage"])
    ap.add_argument("--nodes", type=int, default=111_000_000)
    ap.add_argument("--edges", type=int, default=1_600_000_000, help="edges drawn before symmetrising")
    ap.add_argument("--in-channels", type=int, default=128)
    ap.add_argument("--hidden", type=int, default=256)
    ap.add_argument("--out-channels", type=int, default=172)
    ap.add_argument("--layers", type=int, default=3)
    ap.add_argument("--bits", type=int, default=2)
    ap.add_argument("--pre", type=int, default=0)
    ap.add_argument("--epochs", type=int, default=6)
    ap.add_argument("--train-frac", type=float, default=0.01)
    ap.add_argument("--dropout", type=float, default=0.5)
    ap.add_argument("--lean-halo", type=int, default=1,
                    help="packed halo modes: no fp32 staging buffers (they are tens of GB per GPU at this scale)")
    ap.add_argument("--seed", type=int, default=20261130)
    ap.add_argument("--dense", default="tf32x3", choices=["tf32x3", "cublas"],
                    help="the layers' fp32 transforms: tensor-core kernel (three TF32 products per fp32 product, fp32 "
                         "accumulate) or cuBLAS fp32 SIMT kernels")
    ap.add_argument("--kernel-table", default="",
                    help="after the timed epochs, run one more under torch.profiler and write rank 0's per-kernel "
                         "device-time table to this file (a breakdown, never a timing)")
    ap.add_argument("--transport", default="all_to_all", choices=["all_to_all", "push"],
                    help="halo exchange: one NCCL collective per aggregation, or rows stored straight into the receivers' buffers")
    ap.add_argument("--push-engine", default="auto", choices=["kernel", "copy", "auto"],
                    help="push transport: rows moved by the store kernel, or by device-to-device copies")
    return ap


def run(args):
    """One measurement; returns the result line (a dict) on rank 0, None elsewhere.  Joins the process group that
    is already there (bench.py's multi-GPU leg calls this in-process) or starts one under torchrun."""
    dense.MODE = args.dense
    multi = int(os.environ.get("WORLD_SIZE", "1")) > 1
    comm = Communicator(args.bits, is_async=True, transport=args.transport if multi else "all_to_all",
                        push_engine=args.push_engine)
    if "RANK" in os.environ:
        rank, world = comm.init_dist_group("nccl")
    else:
        rank, world = 0, 1
        torch.cuda.set_device(0)
    device = torch.device("cuda", torch.cuda.current_device())
    torch.cuda.reset_peak_memory_stats()
    Quantizer_for_all_procs(world, args.bits)
    t0 = time.time()
    src, dst, begin = graphgen.partitioned_in_edges("chung_lu", args.nodes, args.edges, args.seed, rank, world, device,
                                                    relabel=True)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    nnz_rank = int(local.shape[1] + remote.shape[1])
    del src, dst
    dims = [args.in_channels] + [args.hidden] * (args.layers - 1) + [args.out_channels]
    lean = bool(args.lean_halo) and args.bits in (2, 4, 8) and world > 1
    graph = build_graph(local, remote, begin, rank, world, max(dims), args.bits, bool(args.pre), device=device,
                        lean_halo=lean)
    del local, remote
    torch.cuda.empty_cache()
    n = graph.local_adj_t.sparse_size(0)
    g = torch.Generator(device=device).manual_seed(args.seed + 17 * rank)
    data = {
        "graph": graph,
        # rows padded to a multiple of 32 floats: every gathered feature row starts on a 128-byte line
        "nodes_features": torch.randn(n, (args.in_channels + 31) // 32 * 32, device=device,
                                      generator=g)[:, :args.in_channels],
        "nodes_labels": torch.randint(0, args.out_channels, (n,), device=device, generator=g),
        "nodes_train_masks": torch.nonzero(torch.rand(n, device=device, generator=g) < args.train_frac).view(-1),
        "nodes_valid_masks": torch.zeros(0, dtype=torch.int64, device=device),
        "nodes_test_masks": torch.zeros(0, dtype=torch.int64, device=device),
    }
    cfg = dict(model_name=args.model, in_channels=args.in_channels, hidden_channels=args.hidden,
               out_channels=args.out_channels, num_layers=args.layers, dropout=args.dropout, lr=0.01, weight_decay=0.0,
               num_bits=args.bits, is_pre_delay=bool(args.pre))
    set_random_seed(args.seed)
    model, optimizer = create_model_and_optimizer(cfg, device)
    TimeRecorder(args.layers, args.epochs, enabled=False)
    torch.cuda.synchronize()
    setup_s = time.time() - t0
    losses, times = train(model, data, optimizer, args.epochs, args.bits, eval_every_epoch=False, log=None)
    dense.check_status()  # raises if a tensor-core kernel gave up on one of its bounded waits
    t = torch.tensor([sum(times[1:]) / max(len(times) - 1, 1), float(nnz_rank),
                      float(sum(graph.comm_splits.send_splits)), torch.cuda.max_memory_allocated() / 2 ** 30],
                     dtype=torch.float64, device=device)
    tmax, tsum = t.clone(), t.clone()
    if world > 1:
        dist.all_reduce(tmax, op=dist.ReduceOp.MAX)
        dist.all_reduce(tsum, op=dist.ReduceOp.SUM)
    result = None
    if rank == 0:
        passes = aggregation_passes(args.model, dims)
        epoch_s = float(tmax[0])
        result = ({
            "metric": "epoch_time", "value": epoch_s, "unit": "s", "higher_is_better": False, "n_gpus": world,
            "aggregated_edges_per_s": float(tsum[1]) * passes / epoch_s, "aggregation_passes_per_step": passes,
            "config": {"model": args.model, "dims": dims, "nodes": args.nodes, "directed_edges_after_symmetrising":
                       int(tsum[1]), "halo": f"{args.bits}-bit" + (" pre/post" if args.pre else "") + (", no fp32 staging buffers" if lean else ""),
                       "halo_rows_sent_per_exchange": int(tsum[2]), "graph": "Chung-Lu gamma=2.1, relabelled",
                       "epochs_timed": len(times) - 1, "dropout": args.dropout, "optimizer": "Adam lr 0.01",
                       "exchange": comm.transport,
                       "dense": ("tcgen05, 3 TF32 products per fp32 product, fp32 accumulate" if args.dense == "tf32x3"
                                 else "cuBLAS fp32")},
            "losses": [round(x, 5) for x in losses], "epoch_times_s": [round(x, 4) for x in times],
            "peak_mem_gib_max_rank": float(tmax[3]), "setup_s": round(setup_s, 1), "data": "synthetic",
        })
    if args.kernel_table:
        from torch.profiler import ProfilerActivity, profile

        TimeRecorder(args.layers, 1, enabled=False)
        with profile(activities=[ProfilerActivity.CUDA]) as prof:
            train(model, data, optimizer, 1, args.bits, eval_every_epoch=False, log=None)
            torch.cuda.synchronize()
        if rank == 0:
            with open(args.kernel_table, "w") as fh:
                fh.write(prof.key_averages().table(sort_by="cuda_time_total", row_limit=60, max_name_column_width=90))
    del model, optimizer, data, graph
    torch.cuda.empty_cache()
    return result


def main():
    args = make_parser().parse_args()
    result = run(args)
    if result is not None:
        print(json.dumps(result), flush=True)
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
