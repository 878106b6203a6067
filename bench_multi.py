"""Multi-GPU leg of bench.py: distributed aggregation on N GPUs of one node (one process per GPU).

Workload "aggregate_rmat22_per_gpu" (weak scaling): R-MAT with 2^22 vertices per GPU (scale
22 + log2 N), edge factor 16, symmetrised, deduplicated, self-loops, vertex ids randomly relabelled,
N contiguous partitions -- the reference's 1-D partitioning across MPI ranks.  Every rank generates
the edge stream from the same seed and keeps the in-edges of its own vertex range, so the global
graph is never held by one process.  One step = Aggregator forward + backward at F = 32, 128, 256:
halo rows gathered and stored straight into the receivers' buffers (or gathered into a staging buffer
and exchanged with one NCCL all-to-all: --exchange all_to_all), local SpMM meanwhile, remote SpMM on
arrival; backward the transposed chain with the deterministic scatter-add.  Adjacency values are
GCN-normalised (d_dst^-1/2 d_src^-1/2; remote degrees fetched once with the halo exchange itself).

Before anything is timed the exchange path is checked on a small instance (`check` in the JSON line);
after the aggregation legs the full-batch epoch times of BASELINE configurations 4 and 5 are measured
on the same GPUs (`epoch`).
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


def run_check(comm, rank, world, device, args):
    """Correctness of the exchange path as it runs here (real NCCL / peer stores, real overlap), on a small
    instance of the benchmark's graph family (2^14 vertices per GPU), before anything is timed.

      fp32 halo   every rank's forward output and input gradient against A.X / A^T.G computed in fp64 with
                  plain torch ops from the global edge list: error relative to sum |a||x| of the row;
      2-bit halo  and pre/post plan: the overlapped run against the same aggregation done without any
                  overlap (blocking all-to-all, device synchronised after every call): bit for bit, plus a
                  checksum of the codes both runs put on the wire; and the 2-bit result against the exact
                  product within the quantisation bound (half a step of every halo row it sums).
    Returns the `check` record of the JSON line; `ok` false makes the benchmark exit non-zero."""
    import torch.distributed as dist

    from gnn_benchmark_b200 import Quantizer_for_all_procs, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    scale = 14 + int(math.ceil(math.log2(world)))
    n, F = 1 << scale, 128
    s, d = graphgen.rmat_edges(scale, 16, seed=77, device=device)
    s, d = graphgen.symmetrize(s, d, n)
    s, d = graphgen.relabel(s, d, n, seed=78)
    begin = graphgen.contiguous_partitions(n, world)
    b0, b1 = int(begin[rank]), int(begin[rank + 1])
    g = torch.Generator(device=device).manual_seed(79)  # same stream on every rank: global operands
    X = torch.randn(n, F, device=device, generator=g)
    G = torch.randn(n, F, device=device, generator=g)
    local, remote = graphgen.partition_edges(s, d, begin, rank)

    def run(bits, is_pre, overlapped):
        saved = (comm.num_bits, comm.transport, comm.is_async)
        comm.num_bits = bits
        if not overlapped:
            comm.transport, comm.is_async = "all_to_all", False
        Quantizer_for_all_procs(world, bits if bits in (2, 4, 8) else 2)
        graph = build_graph(local, remote, begin, rank, world, F, bits if bits in (2, 4, 8) else 2, is_pre, device=device)
        ctx = SimpleNamespace()
        out = Aggregator.forward(ctx, graph, X[b0:b1].contiguous(), 0, bits, is_pre, True)
        if not overlapped:
            torch.cuda.synchronize()
        codes = 0
        if bits != 32:
            codes = int(graph.comm_buf_for_quantization.quantized_send_data_buf.to(torch.int64).sum())
        grad = Aggregator.backward(ctx, G[b0:b1].contiguous())[1]
        torch.cuda.synchronize()
        comm.num_bits, comm.transport, comm.is_async = saved
        return out, grad, codes

    res = {}
    # fp32 against the global product in fp64
    out, grad, _ = run(32, False, True)
    A_dst, A_src = d, s  # edge (src -> dst): out[dst] += x[src]
    want_out = torch.zeros(n, F, dtype=torch.float64, device=device).index_add_(0, A_dst, X.double()[A_src])[b0:b1]
    want_grad = torch.zeros(n, F, dtype=torch.float64, device=device).index_add_(0, A_src, G.double()[A_dst])[b0:b1]
    sc_out = torch.zeros(n, F, dtype=torch.float64, device=device).index_add_(0, A_dst, X.double().abs()[A_src])[b0:b1]
    sc_grad = torch.zeros(n, F, dtype=torch.float64, device=device).index_add_(0, A_src, G.double().abs()[A_dst])[b0:b1]
    err = max(float(((out.double() - want_out).abs() / sc_out.clamp(min=1e-30)).max()),
              float(((grad.double() - want_grad).abs() / sc_grad.clamp(min=1e-30)).max()))
    # 2-bit halo and the pre/post plan: overlapped run == run without overlap
    same = {}
    sums = {}
    for name, bits, is_pre in (("int2", 2, False), ("pre_post_fp32", 32, True), ("pre_post_int2", 2, True)):
        a = run(bits, is_pre, True)
        b = run(bits, is_pre, False)
        same[name] = bool(torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and a[2] == b[2])
        sums[name] = a[2]
        if name == "int2":
            # against the exact product: every halo element is off by at most half a quantisation step of its
            # row (range / 6) plus the bf16 rounding of the row's zero point and scale (2^-8 relative each)
            lo, hi = X.double().min(1).values, X.double().max(1).values
            step = (hi - lo) / 6 + (lo.abs() + (hi - lo)) * 2.0 ** -8
            halo = (A_src < b0) | (A_src >= b1)
            bound = torch.zeros(n, dtype=torch.float64, device=device).index_add_(0, A_dst[halo], step[A_src[halo]])[b0:b1]
            excess = ((a[0].double() - want_out).abs() - bound.unsqueeze(1) - 1e-5 * sc_out).max()
            q_err = float(excess.clamp(min=0))
    stats = torch.tensor([err, q_err] + [0.0 if v else 1.0 for v in same.values()], dtype=torch.float64, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.MAX)
    total = torch.tensor([float(sums["int2"])], dtype=torch.float64, device=device)
    dist.all_reduce(total, op=dist.ReduceOp.SUM)
    ok = bool(stats[0] <= 1e-5 and stats[1] == 0.0 and float(stats[2:].max()) == 0.0)
    res = {"instance": f"R-MAT scale {scale}, {world} partitions, F={F}", "fp32_max_rel_err": float(stats[0]),
           "int2_excess_over_quantisation_bound": float(stats[1]),
           "overlapped_equals_unoverlapped": {k: bool(stats[2 + i] == 0.0) for i, k in enumerate(same)},
           "int2_codes_checksum": int(total.item()), "ok": ok}
    return res


def _timed_steps(step, steps, device):
    """ms per step, max over ranks, CUDA events between barriers."""
    torch.cuda.synchronize()
    dist.barrier()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    torch.cuda.synchronize()
    dist.barrier()
    t = torch.tensor([a.elapsed_time(b) / steps], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


class _NoExchange(object):
    """Context: the same step with the stores and signals of the push transport left out (outputs are then
    meaningless).  The difference to the full step is the exchange time that is NOT hidden behind compute."""

    class _Done(object):
        def wait(self):
            return True

    def __init__(self, plan):
        self.plan = plan

    def __enter__(self):
        self.push, self.signal = self.plan.push, self.plan.peers.signal
        self.plan.push = lambda *a, **k: None
        self.plan.peers.signal = lambda: _NoExchange._Done()

    def __exit__(self, *a):
        self.plan.push, self.plan.peers.signal = self.push, self.signal


def _epoch_legs(args, world):
    """Full-batch epoch time (the other half of the metric) on this job's GPUs: BASELINE configuration 4
    (products-shaped 3-layer GraphSAGE, the whole graph cut into `world` partitions: strong scaling) and
    configuration 5 (papers100M-shaped 3-layer GCN, 2-bit halo) with 111 M / 8 vertices per GPU -- the full
    configuration at 8 GPUs, the same per-GPU load below (the full graph does not fit 4 GPUs)."""
    import bench_epoch

    transport = "push" if args.exchange == "pipelined" else "all_to_all"
    legs = {}
    runs = [
        ("config4_sage_fp32", ["--model", "sage", "--nodes", "2450000", "--edges", "61900000", "--in-channels", "100",
                               "--hidden", "256", "--out-channels", "47", "--train-frac", "0.08", "--bits", "32", "--epochs", "5"]),
        ("config4_sage_int2", ["--model", "sage", "--nodes", "2450000", "--edges", "61900000", "--in-channels", "100",
                               "--hidden", "256", "--out-channels", "47", "--train-frac", "0.08", "--bits", "2", "--epochs", "5",
                               "--lean-halo", "0"]),  # memory is no issue here: keep the fp32 halo buffers (faster kernels)
        ("config5_gcn_int2", ["--model", "gcn", "--nodes", str(111_000_000 * world // 8), "--edges",
                              str(1_600_000_000 * world // 8), "--in-channels", "128", "--hidden", "256", "--out-channels",
                              "172", "--train-frac", "0.01", "--bits", "2", "--epochs", "4"]),
    ]
    for name, argv in runs:
        try:
            r = bench_epoch.run(bench_epoch.make_parser().parse_args(argv + ["--transport", transport, "--push-engine", args.push_engine]))
            if r is not None:
                legs[name] = {"epoch_s": r["value"], "aggregated_edges_per_s": r["aggregated_edges_per_s"],
                              "aggregation_passes_per_step": r["aggregation_passes_per_step"], "config": r["config"],
                              "losses": r["losses"], "peak_mem_gib_max_rank": r["peak_mem_gib_max_rank"],
                              "setup_s": r["setup_s"]}
        except Exception as exc:  # the aggregation line above must not depend on these legs
            legs[name] = {"error": repr(exc)[:300]}
            torch.cuda.empty_cache()
    return legs


def run_multi_gpu(args):
    import benchlib as bench
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.aggregator import Aggregator, gather_rows
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph

    num_bits, is_pre = args.bits, bool(args.pre)
    transport = "push" if args.exchange == "pipelined" else "all_to_all"
    comm = Communicator(num_bits, is_async=True, transport=transport, push_groups=7, push_engine=args.push_engine)
    rank, world = comm.init_dist_group("nccl")
    device = torch.device("cuda", torch.cuda.current_device())
    TimeRecorder(1, 1, enabled=False)
    widths = args.widths
    scale = args.scale + int(math.ceil(math.log2(world)))

    check = None
    if not args.no_check:
        check = run_check(comm, rank, world, device, args)
        if not check["ok"]:
            if rank == 0:
                print(json.dumps({"metric": "aggregated_edges_per_s", "value": None, "n_gpus": world, "check": check,
                                  "error": "the exchange path failed its correctness check; nothing was timed"}), flush=True)
            dist.barrier()
            dist.destroy_process_group()
            raise SystemExit(1)
        torch.cuda.empty_cache()

    # the graph always carries the packed-halo buffers, so the 2-bit variant can be timed on it too
    plan_bits = num_bits if num_bits in (2, 4, 8) else 2
    Quantizer_for_all_procs(world, plan_bits)
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

    def make_step(bits):
        def step():
            for F in widths:
                ctx = SimpleNamespace()
                Aggregator.forward(ctx, graph, X[F], 0, bits, is_pre, True)
                Aggregator.backward(ctx, G[F])
        return step

    def time_variant(bits, steps=3, exchange=None):
        """ms per step (max over ranks) with another halo format / exchange on the same graph."""
        saved = (comm.num_bits, comm.transport)
        comm.num_bits = bits
        if exchange is not None:
            comm.transport = exchange
        step = make_step(bits)
        for _ in range(2):
            step()
        ms = _timed_steps(step, steps, device)
        comm.num_bits, comm.transport = saved
        return ms

    step = make_step(num_bits)
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    with bench.ClockSampler(torch.cuda.current_device()) as clk:
        t_step = _timed_steps(step, args.steps, device) / 1e3
    stats = torch.tensor([float(nnz), float(sum(graph.comm_splits.send_splits)), float(sum(graph.comm_splits.recv_splits))],
                         dtype=torch.float64, device=device)
    dist.all_reduce(stats, op=dist.ReduceOp.SUM)
    nnz_total = float(stats[0].item())
    edges_per_step = 2 * len(widths) * nnz_total

    # how much of the exchange is NOT hidden behind compute, and what the links carry
    exposed = nv = None
    plan = getattr(graph, "push_plan", None)
    if plan is not None:
        with _NoExchange(plan):
            compute_ms = _timed_steps(step, 3, device)
        exposed = {"ms_per_step": t_step * 1e3 - compute_ms, "compute_only_ms_per_step": compute_ms,
                   "how": "step time minus the same step with the stores and signals left out"}
        if num_bits == 32 and not is_pre:
            F = max(widths)
            graph.comm_buf.resize_buffer(graph.comm_splits, F, 32)

            def exchange_only():
                if plan.peers.engine == "copy":
                    gather_rows(X[F], graph.idx_nodes_send_to_others_i32, graph.comm_buf.send_buf)
                    plan.push("forward", "rows", graph.comm_buf.send_buf, 4 * F, (rank + 1) % world, world - 1)
                else:
                    plan.push("forward", "rows", X[F], 4 * F, (rank + 1) % world, world - 1,
                              graph.idx_nodes_send_to_others_i32)
                plan.peers.signal().wait()

            exchange_only()
            ms = _timed_steps(exchange_only, 5, device)
            sent = torch.tensor([float(max(sum(graph.comm_splits.send_splits), sum(graph.comm_splits.recv_splits)) * F * 4)],
                                dtype=torch.float64, device=device)
            dist.all_reduce(sent, op=dist.ReduceOp.MAX)
            gbs = float(sent.item()) / (ms / 1e3) / 1e9
            nv = {"exchange_ms": ms, "bytes_per_rank_per_direction": int(sent.item()), "achieved_gbs": gbs,
                  "frac_of_measured_770": gbs / 770.0, "frac_of_nominal_900": gbs / 900.0, "F": F,
                  "what": "gather + store of all halo rows into the peers' buffers + signal, nothing else running",
                  "engine": plan.peers.engine}

    variants = {}
    if world > 1 and num_bits == 32:
        ms2 = time_variant(2)
        variants["int2_halo"] = {"ms_per_step": ms2, "value": edges_per_step / (ms2 / 1e3), "unit": "edges/s",
                                 "note": "per-row min/max 2-bit codes + bf16 parameters on the wire (the reference's "
                                         "quantised mode); pack fused into the gather / the transposed SpMM, unpack fused "
                                         "into the receive-side SpMM"}
    if plan is not None:
        notes = {"copy": "rows gathered into the send buffer where needed, then one device-to-device copy per peer on "
                         "the copy engines",
                 "kernel": "rows stored into the peers' buffers by the store kernel, gather fused in",
                 "auto": "forward: store kernel with the gather fused in; backward (blocks already contiguous): one "
                         "device-to-device copy per peer"}
        mine = plan.peers.engine
        for other in ("kernel", "copy", "auto"):
            if other == mine:
                continue
            plan.peers.engine = other
            ms_o = time_variant(num_bits)
            ms_o2 = time_variant(2) if num_bits == 32 else None
            variants["push_engine_" + other] = {"ms_per_step": ms_o, "value": edges_per_step / (ms_o / 1e3),
                                                "unit": "edges/s", "int2_halo_ms_per_step": ms_o2, "note": notes[other]}
        plan.peers.engine = mine
        if num_bits == 32 and not is_pre:  # how finely the peers are grouped (fp32 halo, plain plan only)
            mine_g = comm.push_groups
            for g in sorted({1, 2, 3, 4, world - 1}):
                if g == min(mine_g, world - 1) or g > world - 1:
                    continue
                comm.push_groups = g
                ms_g = time_variant(num_bits)
                variants[f"push_groups_{g}"] = {"ms_per_step": ms_g, "value": edges_per_step / (ms_g / 1e3), "unit": "edges/s",
                                                "note": f"peers served in {g} group(s) instead of {min(mine_g, world - 1)}"}
            comm.push_groups = mine_g
        ms_a2a = time_variant(num_bits, exchange="all_to_all")
        variants["nccl_all_to_all"] = {"ms_per_step": ms_a2a, "value": edges_per_step / (ms_a2a / 1e3), "unit": "edges/s",
                                       "note": "same graph and kernels, one NCCL all-to-all per aggregation instead of "
                                               "direct stores (send-side gather into a staging buffer)"}
    e2e = None if args.no_e2e else _run_e2e(args, graph, widths, num_bits, is_pre, n, nnz_total, device)
    clocks = clk.summary()
    halo_rows = int(stats[1].item())
    del graph, X, G, plan
    torch.cuda.empty_cache()
    epochs = None if args.no_epoch else _epoch_legs(args, world)
    if rank == 0:
        peak, peak_kind = bench.measured_peak_gbs()
        cfg = bench.workload_config(world, args.scale, widths)
        cfg.update({"rows_per_gpu": n, "nnz_total": int(nnz_total), "partitions": world,
                    "halo_rows_sent_total": halo_rows, "halo": f"{num_bits}-bit" + (" pre/post" if is_pre else ""),
                    "exchange": ({"kernel": "rows stored straight into the receivers' buffers (gnnagg_push_rows)",
                                  "copy": "rows gathered, then copied straight into the receivers' buffers "
                                          "(gnnagg_push_block, copy engines)",
                                  "auto": "forward rows stored straight into the receivers' buffers by the kernel that "
                                          "gathers them (gnnagg_push_rows), backward blocks copied there "
                                          "(gnnagg_push_block, copy engines)"}[comm.push_engine]
                                 + f", peers served in {min(comm.push_groups, world - 1)} groups, each aggregated on arrival"
                                 if transport == "push" else "one NCCL all-to-all per aggregation"),
                    "setup_s": round(setup_s, 1), "parallelism": f"1-D vertex partition x{world}"})
        by = sum(bench.spmm_algorithmic_bytes(n, nnz, F) for F in widths) * 2
        launches_per_call = 2 * 2 + (1 if transport == "push" else 1)  # local + remote SpMM (chunk + fix-up), store / gather
        line = {
            "metric": "aggregated_edges_per_s", "value": edges_per_step / t_step, "unit": "edges/s", "n_gpus": world,
            "steps": args.steps, "warmup": warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
            "value_int2_halo": variants.get("int2_halo", {}).get("value"),
            "check": check, "clocks": clocks, "e2e": e2e,
            "gpu_launches": args.steps * len(widths) * 2 * launches_per_call,
            "roofline": {"bound": "hbm", "kernel": "spmm_chunk_kernel (all SpMM calls of a step, rank 0)",
                         "achieved": by / t_step / 1e9, "peak": peak, "unit": "GB/s", "frac": by / t_step / 1e9 / peak,
                         "frac_is": "algorithmic SpMM bytes of rank 0 / whole step time (exchange included) / peak",
                         "peak_kind": peak_kind + " copy bandwidth", "traffic": None},
            "exposed_exchange": exposed, "nvlink": nv, "variants": variants, "cpu_baseline": None, "epoch": epochs,
        }
        print(json.dumps(line), flush=True)
    dist.barrier()
    dist.destroy_process_group()
