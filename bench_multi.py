"""Multi-GPU leg of bench.py: distributed aggregation on N GPUs of one node (one process per GPU).

Workload "aggregate_rmat22_per_gpu" (weak scaling): R-MAT with 2^22 vertices per GPU (scale
22 + log2 N), edge factor 16, symmetrised, deduplicated, self-loops, vertex ids randomly relabelled,
N contiguous partitions -- the reference's 1-D partitioning across MPI ranks.  Every rank generates
the edge stream from the same seed and keeps the in-edges of its own vertex range, so the global
graph is never held by one process.  One step = Aggregator forward + backward at F = 32, 128, 256:
send-side gather, halo all-to-all over NCCL overlapped with the local SpMM, remote SpMM; backward the
transposed chain with the deterministic scatter-add.  Adjacency values are GCN-normalised
(d_dst^-1/2 d_src^-1/2; remote degrees fetched once with the halo exchange itself).
"""
import json
import math
import os
import time
from types import SimpleNamespace

import torch
import torch.distributed as dist


def _gcn_values(graph, comm, world):
    """d_dst^-1/2 * d_src^-1/2 on the local and remote matrices; the remote sources' degrees come
    through one fp32 halo exchange of a single column."""
    import torch

    from gnn_benchmark_b200.aggregator import gather_rows

    n = graph.local_adj_t.sparse_size(0)
    dev = graph.local_adj_t.device
    rp_l, col_l, _ = graph.local_adj_t.csr()
    deg = (rp_l[1:] - rp_l[:-1]).to(torch.float32)
    if world > 1:
        rp_r, col_r, _ = graph.remote_adj_t.csr()
        deg = deg + (rp_r[1:] - rp_r[:-1]).to(torch.float32)
    dinv = deg.clamp(min=1).rsqrt()
    rows_l = torch.repeat_interleave(torch.arange(n, device=dev), rp_l[1:] - rp_l[:-1])
    graph.local_adj_t.set_value_(dinv[rows_l] * dinv[col_l.to(torch.int64)])
    if world > 1:
        graph.comm_buf.resize_buffer(graph.comm_splits, 4, 32)
        send = graph.comm_buf.send_buf
        x = dinv.view(-1, 1).expand(n, 4).contiguous()
        gather_rows(x, graph.idx_nodes_send_to_others_i32, send)
        h = comm.comm_with_fp32(graph.comm_splits, graph.comm_buf, "forward")
        if h is not None:
            h.wait()
        torch.cuda.synchronize()
        dinv_halo = graph.comm_buf.recv_buf[:, 0].clone()
        rows_r = torch.repeat_interleave(torch.arange(n, device=dev), rp_r[1:] - rp_r[:-1])
        graph.remote_adj_t.set_value_(dinv[rows_r] * dinv_halo[col_r.to(torch.int64)])


def _run_e2e(args, graph, widths, num_bits, is_pre, n, nnz_total, device):
    """The same step through Aggregator with this rank's features and output gradients in pinned
    HOST memory: per call copy the operand host->device, run, copy the result device->host, pipelined
    over three streams (bench.HostPipeline)."""
    import benchlib as bench
    from gnn_benchmark_b200.aggregator import Aggregator

    Fmax = max(widths)
    host_in = torch.empty(n, Fmax, pin_memory=True).normal_(generator=torch.Generator().manual_seed(1))
    host_out = torch.empty(n, Fmax, pin_memory=True)
    pipe = bench.HostPipeline(device, n * Fmax)

    def step():
        pipe.h2d = pipe.d2h = 0
        for F in widths:
            hin = host_in.view(-1)[: n * F].view(n, F)
            hout = host_out.view(-1)[: n * F].view(n, F)
            ctx = SimpleNamespace()
            pipe.call(hin, hout, (n, F), lambda x, y: Aggregator.forward(ctx, graph, x, 0, num_bits, is_pre, True))
            pipe.call(hin, hout, (n, F), lambda x, y: Aggregator.backward(ctx, x)[1])

    step()
    pipe.drain()
    torch.cuda.synchronize()
    dist.barrier()
    steps = max(1, min(args.steps, 3))
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(pipe.s_in):
        e0.record()
    for _ in range(steps):
        step()
    pipe.drain()
    with torch.cuda.stream(pipe.s_out):
        e1.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([e0.elapsed_time(e1) / 1e3 / steps], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    b = torch.tensor([float(pipe.h2d)], dtype=torch.float64, device=device)
    dist.all_reduce(b, op=dist.ReduceOp.SUM)
    del host_in, host_out, pipe
    return {"value": 2 * len(widths) * nnz_total / float(t.item()), "unit": "edges/s",
            "h2d_bytes_per_step": int(b.item()), "d2h_bytes_per_step": int(b.item()),
            "ms_per_step": float(t.item()) * 1e3, "steps": steps,
            "pipeline": "h2d / kernels / d2h on three streams, two buffer pairs"}


def run_multi_gpu(args):
    import benchlib as bench
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    num_bits = int(os.environ.get("GNNAGG_BENCH_BITS", "32"))  # halo format of the headline number
    is_pre = os.environ.get("GNNAGG_BENCH_PRE", "0") == "1"
    # GNNAGG_BENCH_PIPELINE=1: fp32 halo exchanged peer by peer, each peer's rows aggregated on arrival
    # (measured equal to the one-shot all-to-all at 2 and 4 GPUs, so the one-shot exchange is the default)
    pipeline = os.environ.get("GNNAGG_BENCH_PIPELINE", "0") == "1"
    comm = Communicator(num_bits, is_async=True, pipeline_peers=pipeline)
    rank, world = comm.init_dist_group("nccl")
    device = torch.device("cuda", torch.cuda.current_device())
    # the graph always carries the packed-halo buffers, so the 2-bit variant can be timed on it too
    plan_bits = num_bits if num_bits in (2, 4, 8) else 2
    Quantizer_for_all_procs(world, plan_bits)
    TimeRecorder(1, 1, enabled=False)
    widths = bench.WIDTHS
    scale = bench.SCALE + int(math.ceil(math.log2(world)))

    t0 = time.time()
    src, dst, begin = graphgen.partitioned_in_edges("rmat", 1 << scale, bench.EDGE_FACTOR << scale, bench.SEED, rank, world,
                                                    device, relabel=world > 1, scale=scale)
    local, remote = graphgen.partition_edges(src, dst, begin, rank)
    nnz = int(local.shape[1] + remote.shape[1])  # edges aggregated by this rank per pass
    del src, dst
    graph = build_graph(local, remote, begin, rank, world, max(widths), plan_bits, is_pre, device=device)
    del local, remote
    torch.cuda.empty_cache()
    if not is_pre:
        _gcn_values(graph, comm, world)
    n = graph.local_adj_t.sparse_size(0)
    torch.cuda.synchronize()
    setup_s = time.time() - t0

    g = torch.Generator(device=device).manual_seed(bench.SEED + rank)
    X = {F: torch.randn(n, F, device=device, generator=g) for F in widths}
    G = {F: torch.randn(n, F, device=device, generator=g) for F in widths}

    def step(bits=num_bits):
        for F in widths:
            ctx = SimpleNamespace()
            Aggregator.forward(ctx, graph, X[F], 0, bits, is_pre, True)
            Aggregator.backward(ctx, G[F])

    def time_variant(bits, steps=3):
        """ms per step (max over ranks) with another halo format on the same graph."""
        comm.num_bits = bits
        for _ in range(2):
            step(bits)
        torch.cuda.synchronize()
        dist.barrier()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step(bits)
        b.record()
        torch.cuda.synchronize()
        dist.barrier()
        t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        comm.num_bits = num_bits
        return float(t.item())

    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    with bench.ClockSampler(torch.cuda.current_device()) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
    t_local = e0.elapsed_time(e1) / 1e3 / args.steps
    stats = torch.tensor([t_local, float(nnz), float(sum(graph.comm_splits.send_splits)),
                          float(sum(graph.comm_splits.recv_splits))], dtype=torch.float64, device=device)
    t_max = stats[0:1].clone()
    dist.all_reduce(t_max, op=dist.ReduceOp.MAX)
    tot = stats.clone()
    dist.all_reduce(tot, op=dist.ReduceOp.SUM)
    t_step = float(t_max.item())
    edges_per_step = 2 * len(widths) * float(tot[1].item())

    # the exchange alone (not overlapped), widest feature, forward direction: NVLink fraction
    nv = None
    if world > 1 and num_bits == 32:
        F = max(widths)
        graph.comm_buf.resize_buffer(graph.comm_splits, F, 32)
        ts = []
        for _ in range(5):
            dist.barrier()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            h = comm.comm_with_fp32(graph.comm_splits, graph.comm_buf, "forward")
            if h is not None:
                h.wait()
            b.record()
            torch.cuda.synchronize()
            ts.append(a.elapsed_time(b) / 1e3)
        t_x = torch.tensor([sorted(ts)[len(ts) // 2]], dtype=torch.float64, device=device)
        dist.all_reduce(t_x, op=dist.ReduceOp.MAX)
        sent = max(sum(graph.comm_splits.send_splits), sum(graph.comm_splits.recv_splits)) * F * 4
        sent_t = torch.tensor([float(sent)], dtype=torch.float64, device=device)
        dist.all_reduce(sent_t, op=dist.ReduceOp.MAX)
        gbs = float(sent_t.item()) / float(t_x.item()) / 1e9
        nv = {"exchange_ms": float(t_x.item()) * 1e3, "bytes_per_rank_per_direction": int(sent_t.item()),
              "achieved_gbs": gbs, "frac_of_measured_770": gbs / 770.0, "frac_of_nominal_900": gbs / 900.0, "F": F}

    variants = None
    if world > 1 and num_bits == 32:
        ms2 = time_variant(2)
        variants = {"int2_halo": {"ms_per_step": ms2, "value": edges_per_step / (ms2 / 1e3), "unit": "edges/s",
                                  "note": "per-row min/max 2-bit codes + bf16 parameters on the wire (the "
                                          "reference's quantised mode), unpack fused into the receive-side SpMM"}}
    e2e = _run_e2e(args, graph, widths, num_bits, is_pre, n, float(tot[1].item()), device)
    clocks = clk.summary()
    if rank == 0:
        peak, peak_kind = bench.measured_peak_gbs()
        cfg = bench.workload_config(world)
        cfg.update({"rows_per_gpu": n, "nnz_total": int(tot[1].item()), "partitions": world,
                    "halo_rows_sent_total": int(tot[2].item()), "halo": f"{num_bits}-bit" + (" pre/post" if is_pre else ""),
                    "exchange": "peer-by-peer, aggregated on arrival" if (pipeline and num_bits == 32 and not is_pre)
                    else "one all-to-all per aggregation",
                    "setup_s": round(setup_s, 1), "parallelism": f"1-D vertex partition x{world}"})
        by = sum(bench.spmm_algorithmic_bytes(n, nnz, F) for F in widths) * 2
        line = {
            "metric": "aggregated_edges_per_s", "value": edges_per_step / t_step, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "clocks": clocks,
            "e2e": e2e,
            "gpu_launches": args.steps * len(widths) * (2 * 2 * (1 if world == 1 else 2) + (1 if world > 1 else 0)),
            "roofline": {"bound": "hbm", "kernel": "spmm_chunk_kernel (all SpMM calls of a step, rank 0)",
                         "achieved": by / t_step / 1e9, "peak": peak, "unit": "GB/s", "frac": by / t_step / 1e9 / peak,
                         "peak_kind": peak_kind + " copy bandwidth", "traffic": None,
                         "note": "whole step including the exchange; SpMM algorithmic bytes only"},
            "nvlink": nv, "variants": variants, "cpu_baseline": None,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
