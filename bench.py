"""Benchmark of the graph-aggregation hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

N = 1  workload "spmm_rmat22": the single-GPU SpMM microbenchmark -- R-MAT scale 22, edge factor
       16, (a,b,c,d) = (.57,.19,.19,.05), symmetrised, deduplicated, self-loops, GCN-normalised
       fp32 CSR values, int32 columns, int64 row pointers; one step = forward A.X and transposed
       A^T.G at feature widths 32, 128 and 256 (six SpMM calls).
N > 1  workload "aggregate_rmat22_per_gpu": the same graph family with 2^22 vertices per GPU,
       randomly relabelled and cut into N contiguous partitions; one step = Aggregator forward +
       backward (halo exchange over NCCL overlapped with the local SpMM) at the same three widths.

Prints ONE JSON line (rank 0).  `value` = aggregated edges per second over the whole job with
inputs resident in HBM; `e2e` = the same metric through the public call with pinned HOST buffers,
H2D/D2H copies inside the timed region; `roofline` = algorithmic bytes of the widest SpMM launch
over its CUDA-event time, against the measured HBM copy bandwidth; `cpu_baseline` = the
reference's own CPU SpMM (compiled from its sources when available, else the C port) timed on
this box's host cores on a stated sample.

--impl reference times only that CPU implementation, same metric and workload, and prints the
same line with "impl": "reference".
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

from benchlib import (EDGE_FACTOR, SCALE, SEED, WIDTHS, ClockSampler, HostPipeline, measured_peak_gbs,  # noqa: E402
                      spmm_algorithmic_bytes, workload_config)

NCU_DRAM_BYTES_PER_LAUNCH = {}

# ------------------------------------------------------------------------------------------------
def build_single_gpu_graph(device):
    from gnn_benchmark_b200 import SparseTensor, graphgen

    n = 1 << SCALE
    s, d = graphgen.rmat_edges(SCALE, EDGE_FACTOR, seed=SEED, device=device)
    s, d = graphgen.symmetrize(s, d, n)
    rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
    del s, d
    A = SparseTensor(rowptr=rowptr, col=col, value=val, sparse_sizes=(n, n))
    A.validate()
    A.storage.colptr()  # CSC twin for the transposed product, built once like the reference caches it
    torch.cuda.empty_cache()
    return A


def cpu_reference_spmm(rowptr, col64, val, X, out, splits, ref_mod):
    """One accumulating SpMM on the host: the reference's compiled kernel, or the C port."""
    import oracle

    if ref_mod is not None:
        M = rowptr.numel() - 1
        ref_mod.spmm(rowptr, col64, val, X, out, M, splits, torch.tensor([0, X.size(1)], dtype=torch.int32))
    else:
        oracle.spmm(rowptr.numpy(), col64.numpy(), val.numpy(), X.numpy(), out.numpy())


class CpuArm:
    """The reference's CPU SpMM on this box's host cores.  Sample = forward + transposed product at
    F = 128 on the full benchmark graph (2 of the 6 calls of a step; 520 of the step's mean 563
    algorithmic bytes per edge)."""
    SAMPLE_F = 128

    def __init__(self, A):
        import oracle

        self.ref_mod = oracle.load_reference_module()
        self.kind = "reference" if self.ref_mod is not None else "port"
        self.cores = torch.get_num_threads() if self.ref_mod is not None else oracle.num_threads()
        rowptr, col, val = A.csr()
        self.fwd = (rowptr.cpu(), col.cpu().to(torch.int64), val.cpu())
        self.bwd = (A.storage.colptr().cpu(), A.storage.row_T().cpu().to(torch.int64), A.storage.value_T().cpu())
        self.nnz = A.nnz()
        n = A.sparse_size(0)
        g = torch.Generator().manual_seed(SEED)
        self.X = torch.randn(n, self.SAMPLE_F, generator=g)
        self.out = torch.zeros(n, self.SAMPLE_F)
        ones = torch.ones(self.nnz)
        self.splits = [torch.from_numpy(oracle.distribute_work_for_row(t[0].numpy(), ones.numpy(), self.cores))
                       for t in (self.fwd, self.bwd)]
        self.sample = (f"forward + transposed SpMM at F={self.SAMPLE_F} on the full R-MAT scale-{SCALE} graph "
                       f"({2 * self.nnz} edges per step)")

    def step(self):
        for (rp, c, v), sp in zip((self.fwd, self.bwd), self.splits):
            cpu_reference_spmm(rp, c, v, self.X, self.out, sp, self.ref_mod)
        return 2 * self.nnz

    def run(self, steps, warmup):
        for _ in range(warmup):
            self.step()
        t0 = time.perf_counter()
        edges = 0
        for _ in range(steps):
            edges += self.step()
        dt = time.perf_counter() - t0
        return edges / dt, dt / steps


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    device = torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")
    A = build_single_gpu_graph(device) if device.type == "cuda" else _cpu_graph()
    arm = CpuArm(A)
    value, sec_per_step = arm.run(args.steps, args.warmup)
    line = {
        "impl": "reference", "metric": "aggregated_edges_per_s", "value": value, "unit": "edges/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus, A),
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": arm.cores, "kind": arm.kind,
                         "sample": arm.sample},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def _cpu_graph():
    from gnn_benchmark_b200 import SparseTensor, graphgen

    n = 1 << SCALE
    s, d = graphgen.rmat_edges(SCALE, EDGE_FACTOR, seed=SEED, device="cpu")
    s, d = graphgen.symmetrize(s, d, n)
    rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
    A = SparseTensor(rowptr=rowptr, col=col, value=val, sparse_sizes=(n, n))
    A.storage.colptr()
    return A


# ------------------------------------------------------------------------------------------------
def run_single_gpu(args):
    from gnn_benchmark_b200 import SPMM_backward, SPMM_forward

    device = torch.device("cuda", 0)
    torch.cuda.set_device(device)
    A = build_single_gpu_graph(device)
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
    for _ in range(max(args.warmup, 3)):
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
    per_width = {}
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
        avg = sum(times) / len(times)
        by = spmm_algorithmic_bytes(n, nnz, F)
        per_width[F] = {"ms": avg * 1e3, "algorithmic_bytes": by, "gbs": by / avg / 1e9,
                        "edges_per_s": nnz / avg}
    peak, peak_kind = measured_peak_gbs()
    top = max(WIDTHS, key=lambda F: per_width[F]["ms"])
    roofline = {
        "bound": "hbm", "kernel": f"spmm_chunk_kernel (F={top}, forward and transposed launches averaged)",
        "achieved": per_width[top]["gbs"], "peak": peak, "unit": "GB/s", "frac": per_width[top]["gbs"] / peak,
        "peak_kind": peak_kind + " copy bandwidth, burst",
        "traffic": NCU_DRAM_BYTES_PER_LAUNCH.get(top) if SCALE == 22 else None,
        "traffic_gbs": (NCU_DRAM_BYTES_PER_LAUNCH[top] / (per_width[top]["ms"] / 1e3) / 1e9
                        if SCALE == 22 and top in NCU_DRAM_BYTES_PER_LAUNCH else None),
        "by_width": {str(F): {"ms": round(per_width[F]["ms"], 4), "gbs": round(per_width[F]["gbs"], 1),
                              "frac": round(per_width[F]["gbs"] / peak, 4)} for F in WIDTHS},
    }

    # ---- end to end through the public call with pinned host buffers ----
    e2e = None if args.no_e2e else run_e2e_single(A, args, device)

    # ---- CPU baseline on the host cores ----
    del X, G, Y
    torch.cuda.empty_cache()
    cpu = None
    if not args.no_cpu_baseline:
        arm = CpuArm(A)
        v, _ = arm.run(steps=2, warmup=1)
        cpu = {"value": v, "unit": "edges/s", "cores": arm.cores, "kind": arm.kind, "sample": arm.sample}

    config = workload_config(1, A)
    epoch = None
    if not args.no_epoch:
        del A
        torch.cuda.empty_cache()
        epoch = run_epoch_leg()

    line = {
        "metric": "aggregated_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": 1, "steps": args.steps,
        "warmup": max(args.warmup, 3), "ms_per_step": t_step * 1e3, "higher_is_better": True, "scaling": "weak",
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


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", type=str, default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true", help="skip the host-buffer leg (profiler captures)")
    ap.add_argument("--no-epoch", action="store_true", help="skip the full-batch epoch leg (N = 1 only)")
    args = ap.parse_args()

    if args.impl == "reference":
        run_reference_arm(args)
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
