"""Reference arm of bench.py (`--impl reference`): the reference's own CPU implementation of the path
on this box's host cores, with every thread the process may use, on the same workload family, metric
and unit as the GPU arm.

N = 1  the compiled AVX-512 `spmm` of the reference (oracle/_ref, else the C port) on the full R-MAT
       scale-22 graph; one step = forward + transposed product at F = 128 (a bounded sample of the six
       calls of a GPU step: 2 calls, 520 of the step's mean 563 algorithmic bytes per edge).
N > 1  the reference's partitioned aggregation (plain plan, send-side gather, exchange, local + remote
       SpMM, transposed backward, scatter-add; oracle/aggregate_cpu.py) for all N partitions of the
       GPU arm's graph family at a stated down-scale, emulated by rank 0 alone with all host threads
       (under torchrun the other ranks exit at once); one step = Aggregator forward + backward at
       F = 128 on every partition.  The all-to-all between the emulated ranks is a host-memory copy, so
       the figure is an upper bound of what N MPI ranks sharing these cores would reach.

Nothing here touches the CUDA library: graphs are generated with plain torch ops (on the GPU when there
is one, then moved to the host).
"""
import json
import os
import time

import torch

import benchlib

SAMPLE_F = 128
# vertices per partition of the N > 1 sample: 2^19 instead of the GPU arm's 2^22
MULTI_SCALE_PER_PART = 19


def host_threads() -> int:
    try:
        return len(os.sched_getaffinity(0))
    except AttributeError:
        return os.cpu_count() or 1


def _gen_device():
    return torch.device("cuda", 0) if torch.cuda.is_available() else torch.device("cpu")


def _timed(step, steps, warmup):
    for _ in range(warmup):
        step()
    t0 = time.perf_counter()
    edges = 0
    for _ in range(steps):
        edges += step()
    dt = time.perf_counter() - t0
    return edges / dt, dt / steps


class SpmmArm(object):
    """N = 1: forward + transposed SpMM at F = 128 on the full benchmark graph."""

    def __init__(self, scale, threads):
        import oracle
        from gnn_benchmark_b200 import graphgen

        torch.set_num_threads(threads)
        dev = _gen_device()
        n = 1 << scale
        s, d = graphgen.rmat_edges(scale, benchlib.EDGE_FACTOR, seed=benchlib.SEED, device=dev)
        s, d = graphgen.symmetrize(s, d, n)
        rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
        del s, d
        # transposed operand: stable sort by column keeps rows ascending inside a column
        order = torch.sort(col.to(torch.int64), stable=True)[1]
        rows = torch.repeat_interleave(torch.arange(n, device=dev), rowptr[1:] - rowptr[:-1])
        colptr = torch.zeros(n + 1, dtype=torch.int64, device=dev)
        torch.cumsum(torch.bincount(col.to(torch.int64), minlength=n), 0, out=colptr[1:])
        self.fwd = (rowptr.cpu(), col.cpu().to(torch.int64), val.cpu())
        self.bwd = (colptr.cpu(), rows[order].cpu(), val[order].cpu())
        del rowptr, col, val, order, rows, colptr
        if dev.type == "cuda":
            torch.cuda.empty_cache()
        self.n, self.nnz, self.threads = n, self.fwd[1].numel(), threads
        self.ref = oracle.load_reference_module()
        self.kind = "reference" if self.ref is not None else "port"
        g = torch.Generator().manual_seed(benchlib.SEED)
        self.X = torch.randn(n, SAMPLE_F, generator=g)
        self.out = torch.zeros(n, SAMPLE_F)
        self.splits = [torch.from_numpy(oracle.distribute_work_for_row(t[0].numpy(), t[2].numpy(), threads))
                       for t in (self.fwd, self.bwd)]
        self.sample = (f"forward + transposed SpMM at F={SAMPLE_F} on the full R-MAT scale-{scale} graph "
                       f"({2 * self.nnz} edges per step)")

    def step(self):
        import oracle

        for (rp, c, v), sp in zip((self.fwd, self.bwd), self.splits):
            if self.ref is not None:
                self.ref.spmm(rp, c, v, self.X, self.out, self.n, sp, torch.tensor([0, SAMPLE_F], dtype=torch.int32))
            else:
                oracle.spmm(rp.numpy(), c.numpy(), v.numpy(), self.X.numpy(), self.out.numpy())
        return 2 * self.nnz


class AggregateArm(object):
    """N > 1: all N partitions' Aggregator forward + backward, emulated in one process."""

    def __init__(self, world, threads):
        from gnn_benchmark_b200 import graphgen
        from oracle import aggregate_cpu

        dev = _gen_device()
        self.scale = MULTI_SCALE_PER_PART + (world - 1).bit_length()
        n = 1 << self.scale
        s, d = graphgen.rmat_edges(self.scale, benchlib.EDGE_FACTOR, seed=benchlib.SEED, device=dev)
        s, d = graphgen.symmetrize(s, d, n)
        s, d = graphgen.relabel(s, d, n, seed=benchlib.SEED + 1)
        begin = graphgen.contiguous_partitions(n, world)
        parts = aggregate_cpu.build_partitions(s, d, begin, threads)
        del s, d
        self.agg = aggregate_cpu.CpuAggregator(parts, threads)
        self.kind = self.agg.kind
        g = torch.Generator().manual_seed(benchlib.SEED)
        self.X = [torch.randn(p.n, SAMPLE_F, generator=g) for p in parts]
        self.G = [torch.randn(p.n, SAMPLE_F, generator=g) for p in parts]
        self.rows_per_rank = parts[0].n
        self.nnz_total = self.agg.edges_per_pass()
        self.halo_rows = sum(sum(p.send_splits) for p in parts)
        self.sample = (f"Aggregator forward + backward at F={SAMPLE_F}, fp32 halo, on all {world} partitions of an R-MAT "
                       f"scale-{self.scale} graph (2^{MULTI_SCALE_PER_PART} vertices per partition, the GPU arm has 2^"
                       f"{benchlib.SCALE}), ranks emulated one after the other by one process")

    def step(self):
        self.agg.forward(self.X)
        self.agg.backward(self.G)
        return 2 * self.nnz_total


def run(args):
    if int(os.environ.get("RANK", "0")) != 0:
        return
    world = max(int(os.environ.get("WORLD_SIZE", "1")), args.gpus)
    threads = host_threads()  # torchrun exports OMP_NUM_THREADS=1: the count is set explicitly instead
    t0 = time.time()
    if world == 1:
        arm = SpmmArm(args.scale, threads)
        cfg = benchlib.workload_config(1, args.scale, args.widths)
        cfg.update({"rows": arm.n, "nnz": arm.nnz, "sampled_widths": [SAMPLE_F]})
    else:
        arm = AggregateArm(world, threads)
        cfg = benchlib.workload_config(world, args.scale, args.widths)
        cfg.update({"rows_per_rank": arm.rows_per_rank, "nnz_total": arm.nnz_total, "partitions": world,
                    "halo_rows_sent_total": arm.halo_rows, "halo": "32-bit", "sampled_widths": [SAMPLE_F],
                    "scale_factor": 2.0 ** (MULTI_SCALE_PER_PART - args.scale), "threads_per_rank": threads,
                    "ranks": "emulated in one process, exchange = host-memory copy"})
    setup_s = time.time() - t0
    value, sec_per_step = _timed(arm.step, args.steps, min(args.warmup, 1) if world > 1 else args.warmup)
    cfg["setup_s"] = round(setup_s, 1)
    line = {
        "impl": "reference", "metric": "aggregated_edges_per_s", "value": value, "unit": "edges/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": sec_per_step * 1e3, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic", "config": cfg,
        "cpu_baseline": {"value": value, "unit": "edges/s", "cores": threads, "kind": arm.kind, "sample": arm.sample},
        "e2e": {"value": value, "unit": "edges/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
