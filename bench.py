"""Benchmark of the graph-aggregation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--scale S] [--widths 32,128,256]

N = 1  workload "spmm_rmat22": the single-GPU SpMM microbenchmark -- R-MAT scale 22, edge factor
       16, (a,b,c,d) = (.57,.19,.19,.05), symmetrised, deduplicated, self-loops, GCN-normalised
       fp32 CSR values, int32 columns, int64 row pointers; one step = forward A.X and transposed
       A^T.G at feature widths 32, 128 and 256 (six SpMM calls).
N > 1  workload "aggregate_rmat22_per_gpu" (bench_multi.py): the same graph family with 2^22 vertices
       per GPU, randomly relabelled and cut into N contiguous partitions; one step = Aggregator forward
       + backward (halo exchange overlapped with the SpMMs) at the same three widths.

Prints ONE JSON line (rank 0).  `value` = aggregated edges per second over the whole job with
inputs resident in HBM; `e2e` = the same metric through the public call with pinned HOST buffers,
H2D/D2H copies inside the timed region; `roofline` = the SpMM launches of the widest feature width:
algorithmic bytes (no-reuse gather model), compulsory bytes and measured DRAM traffic, each over the
CUDA-event time and against the measured HBM copy bandwidth; `cpu_baseline` = the reference's own
CPU SpMM (compiled from its sources when available, else the C port) timed on this box's host cores
on a stated sample; `epoch` = full-batch epoch time of the products-shaped GraphSAGE (bench_epoch.py).

--impl reference (bench_reference.py) times only the reference's CPU implementation, same metric and
workload family, and prints the same line with "impl": "reference".
--scale / --widths choose a smaller case (profiler captures); they are echoed into `config`.
"""
import argparse
import json
import os
import subprocess
import sys
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import benchlib  # noqa: E402
from benchlib import EDGE_FACTOR, SEED, ClockSampler, HostPipeline, measured_peak_gbs  # noqa: E402


def build_single_gpu_graph(device, scale):
    from gnn_benchmark_b200 import SparseTensor, graphgen

    n = 1 << scale
    s, d = graphgen.rmat_edges(scale, EDGE_FACTOR, seed=SEED, device=device)
    s, d = graphgen.symmetrize(s, d, n)
    rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
    del s, d
    A = SparseTensor(rowptr=rowptr, col=col, value=val, sparse_sizes=(n, n))
    A.validate()
    A.storage.colptr()  # CSC twin for the transposed product, built once like the reference caches it
    torch.cuda.empty_cache()
    return A


def run_single_gpu(args):
    from gnn_benchmark_b200 import SPMM_backward, SPMM_forward

    WIDTHS = args.widths
    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    A = build_single_gpu_graph(device, args.scale)
    n, nnz = A.sparse_size(0), A.nnz()
    g = torch.Generator(device=device).manual_seed(SEED)
    X = {F: torch.randn(n, F, device=device, generator=g) for F in WIDTHS}
    G = {F: torch.randn(n, F, device=device, generator=g) for F in WIDTHS}
    Y = {F: torch.empty(n, F, device=device) for F in WIDTHS}

    def step():
        for F in WIDTHS:
            SPMM_forward(A, X[F], Y[F], accumulate=False)
            SPMM_backward(A, G[F], Y[F], accumulate=False)

    launches_per_step = 2 * 2 * len(WIDTHS)  # chunk kernel + fix-up kernel per call
    warmup = max(args.warmup, 3)
    for _ in range(warmup):
        step()
    torch.cuda.synchronize()

    # ---- whole-step timing (value) ----
    with ClockSampler(0) as clk:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        e0.record()
        for _ in range(args.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        # keep the sampler running a moment longer on short runs so that it sees load
        t_step = e0.elapsed_time(e1) / 1e3 / args.steps
        spin_until = time.time() + max(0.0, 1.0 - t_step * args.steps)
        while time.time() < spin_until:
            step()
        torch.cuda.synchronize()
    clocks = clk.summary()
    value = 2 * len(WIDTHS) * nnz / t_step

    # ---- per-launch timing of every width (roofline) ----
    peak, peak_kind = measured_peak_gbs()
    by_width = {}
    for F in WIDTHS:
        times = []
        for fn, src in ((SPMM_forward, X), (SPMM_backward, G)):
            for _ in range(max(3, args.steps)):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                fn(A, src[F], Y[F], accumulate=False)
                b.record()
                torch.cuda.synchronize()
                times.append(a.elapsed_time(b) / 1e3)
        t = sum(times) / len(times)
        alg = benchlib.spmm_algorithmic_bytes(n, nnz, F)
        b_min = benchlib.spmm_compulsory_bytes(n, n, nnz, F)
        traffic = benchlib.spmm_dram_traffic(args.scale, F)
        by_width[F] = {
            "ms": round(t * 1e3, 4), "edges_per_s": nnz / t,
            "algorithmic": alg, "b_min": b_min, "traffic": traffic,
            "algorithmic_gbs": round(alg / t / 1e9, 1), "frac_algorithmic": round(alg / t / 1e9 / peak, 4),
            "frac_b_min": round(b_min / t / 1e9 / peak, 4),
            "traffic_gbs": None if traffic is None else round(traffic / t / 1e9, 1),
            "frac_traffic": None if traffic is None else round(traffic / t / 1e9 / peak, 4),
        }
    top = max(WIDTHS, key=lambda F: by_width[F]["ms"])
    w = by_width[top]
    roofline = {
        "bound": "hbm", "kernel": f"spmm_chunk_kernel (F={top}, forward and transposed launches averaged)",
        "achieved": w["algorithmic"] / (w["ms"] / 1e3) / 1e9, "peak": peak, "unit": "GB/s",
        # the physical fraction: DRAM bytes the launch moved (ncu) over its CUDA-event time; the algorithmic
        # figure counts a gathered row per nonzero and exceeds the peak where L2 serves the hub rows
        "frac": w["frac_traffic"] if w["frac_traffic"] is not None else w["frac_algorithmic"],
        "frac_is": ("dram traffic / event time / peak" if w["frac_traffic"] is not None
                    else "algorithmic bytes / event time / peak (no DRAM capture for this kernel source)"),
        "frac_algorithmic": w["frac_algorithmic"], "frac_b_min": w["frac_b_min"],
        "peak_kind": peak_kind + " copy bandwidth, burst", "traffic": w["traffic"], "b_min": w["b_min"],
        "traffic_source": ("ncu dram__bytes_read.sum + dram__bytes_write.sum of one launch on this workload, kernel "
                           "source " + str(benchlib.SPMM_DRAM_TRAFFIC["kernel_source"])),
        "by_width": {str(F): by_width[F] for F in WIDTHS},
    }

    # ---- end to end through the public call with pinned host buffers ----
    e2e = None if args.no_e2e else run_e2e_single(A, args, device)
    if e2e is not None:
        e2e["note"] = ("bound by the host link: every call moves its dense operand in and its result out over PCIe "
                       "(bytes above), the kernels are a sixth of the step")

    # ---- CPU baseline on the host cores ----
    del X, G, Y
    config = benchlib.workload_config(1, args.scale, WIDTHS, A)
    del A
    torch.cuda.empty_cache()
    cpu = None
    if not args.no_cpu_baseline:
        import bench_reference

        arm = bench_reference.SpmmArm(args.scale, bench_reference.host_threads())
        v, _ = bench_reference._timed(arm.step, 2, 1)
        cpu = {"value": v, "unit": "edges/s", "cores": arm.threads, "kind": arm.kind, "sample": arm.sample}
        del arm

    epoch = None if args.no_epoch else run_epoch_leg()
    line = {
        "metric": "aggregated_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
        "warmup": warmup, "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": config,
        "clocks": clocks, "e2e": e2e, "gpu_launches": launches_per_step * args.steps, "roofline": roofline,
        "cpu_baseline": cpu, "epoch": epoch,
    }
    print(json.dumps(line), flush=True)


def run_epoch_leg():
    """The other half of the metric: full-batch epoch time of the products-shaped 3-layer GraphSAGE
    (2.45 M nodes, 61.9 M undirected Chung-Lu edges, 100 -> 256 -> 256 -> 47) on this GPU, measured by
    `gnn_benchmark_b200.bench_epoch` in a process of its own after this one has released its buffers."""
    cmd = [sys.executable, os.path.join(ROOT, "bench_epoch.py"), "--model", "sage", "--nodes", "2450000",
           "--edges", "61900000", "--in-channels", "100", "--hidden", "256", "--out-channels", "47",
           "--train-frac", "0.08", "--bits", "32", "--epochs", "5"]
    env = {k: v for k, v in os.environ.items() if k not in ("RANK", "LOCAL_RANK", "WORLD_SIZE")}
    try:
        out = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env,
                             cwd=os.path.dirname(os.path.abspath(__file__)))
        lines = [ln for ln in out.stdout.splitlines() if ln.startswith("{")]
        if out.returncode != 0 or not lines:
            return {"error": (out.stderr or out.stdout)[-300:]}
        d = json.loads(lines[-1])
        return {"workload": "sage_chunglu_2.45M_nodes_124M_edges_100-256-256-47", "epoch_s": d["value"],
                "aggregated_edges_per_s": d["aggregated_edges_per_s"],
                "aggregation_passes_per_step": d["aggregation_passes_per_step"], "epochs_timed":
                d["config"]["epochs_timed"], "dense": d["config"]["dense"], "dropout": d["config"]["dropout"]}
    except Exception as exc:  # the SpMM line above must not depend on this leg
        return {"error": repr(exc)[:300]}


def run_e2e_single(A, args, device):
    """SPMM_forward / SPMM_backward with the dense operand in pinned host memory: per call, copy the
    operand host->device, run, copy the result device->host (pipelined over three streams).  The sparse
    matrix (the graph) stays resident, as it does in the reference, which caches it on the SparseTensor."""
    from gnn_benchmark_b200 import SPMM_backward, SPMM_forward

    WIDTHS = args.widths
    n, nnz = A.sparse_size(0), A.nnz()
    Fmax = max(WIDTHS)
    host_in = torch.empty(n, Fmax, pin_memory=True)
    host_in.normal_(generator=torch.Generator().manual_seed(SEED))
    host_out = torch.empty(n, Fmax, pin_memory=True)
    pipe = HostPipeline(device, n * Fmax)

    def step():
        pipe.h2d = pipe.d2h = 0
        for F in WIDTHS:
            hin = host_in.view(-1)[: n * F].view(n, F)
            hout = host_out.view(-1)[: n * F].view(n, F)
            for fn in (SPMM_forward, SPMM_backward):
                def kernel(x, y, fn=fn):
                    fn(A, x, y, accumulate=False)
                    return y
                pipe.call(hin, hout, (n, F), kernel)

    step()
    pipe.drain()
    torch.cuda.synchronize()
    steps = max(1, min(args.steps, 3))
    t0 = time.perf_counter()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    with torch.cuda.stream(pipe.s_in):
        e0.record()
    for _ in range(steps):
        step()
    pipe.drain()
    with torch.cuda.stream(pipe.s_out):
        e1.record()
    torch.cuda.synchronize()
    wall = (time.perf_counter() - t0) / steps
    t = e0.elapsed_time(e1) / 1e3 / steps
    out = {"value": 2 * len(WIDTHS) * nnz / t, "unit": "edges/s", "h2d_bytes_per_step": pipe.h2d,
           "d2h_bytes_per_step": pipe.d2h, "ms_per_step": t * 1e3, "wall_ms_per_step": wall * 1e3, "steps": steps,
           "pipeline": "h2d / kernel / d2h on three streams, two buffer pairs"}
    del host_in, host_out, pipe
    return out


def _widths(text):
    return tuple(int(w) for w in text.split(","))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--scale", type=int, default=benchlib.SCALE,
                    help="log2 of the vertices per GPU (22 is the benchmark; smaller only for profiler captures)")
    ap.add_argument("--widths", type=_widths, default=benchlib.WIDTHS, help="feature widths of a step, comma-separated")
    ap.add_argument("--bits", type=int, default=32, choices=[32, 16, 8, 4, 2],
                    help="N > 1: halo format of the headline value (the 2-bit value is always reported beside it)")
    ap.add_argument("--pre", action="store_true", help="N > 1: pre/post-aggregation plan instead of the plain halo")
    ap.add_argument("--exchange", default="pipelined", choices=["pipelined", "all_to_all"],
                    help="N > 1: peer-by-peer exchange with each peer's rows aggregated on arrival, or one all-to-all")
    ap.add_argument("--push-engine", default="auto", choices=["kernel", "copy", "auto"],
                    help="N > 1, pipelined exchange: rows moved by the store kernel, or by device-to-device copies")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--no-epoch", action="store_true", help="skip the full-batch epoch legs")
    ap.add_argument("--no-check", action="store_true", help="N > 1: skip the correctness check of the exchange path")
    args = ap.parse_args()

    if args.impl == "reference":
        import bench_reference

        bench_reference.run(args)
        return
    from gnn_benchmark_b200 import _lib, build

    build.build()
    _lib.lib()  # fail loudly here if the CUDA library is missing
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the aggregation path has no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    if world > 1 or args.gpus > 1:
        from bench_multi import run_multi_gpu

        run_multi_gpu(args)
    else:
        run_single_gpu(args)


if __name__ == "__main__":
    main()
