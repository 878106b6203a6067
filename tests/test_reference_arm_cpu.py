"""The host-side restatement of the reference's partitioned aggregation (oracle/aggregate_cpu.py, the
CPU baseline of bench.py at more than one GPU) against the global product it must equal."""
import numpy as np
import torch

from gnn_benchmark_b200 import graphgen
from oracle import aggregate_cpu


def test_emulated_ranks_equal_global_product():
    P, scale, F = 4, 10, 16
    n = 1 << scale
    s, d = graphgen.rmat_edges(scale, 8, seed=5, device="cpu")
    s, d = graphgen.symmetrize(s, d, n)
    s, d = graphgen.relabel(s, d, n, seed=6)
    begin = graphgen.contiguous_partitions(n, P)
    parts = aggregate_cpu.build_partitions(s, d, begin, threads=2)
    agg = aggregate_cpu.CpuAggregator(parts, 2)
    g = torch.Generator().manual_seed(1)
    X, G = torch.randn(n, F, generator=g), torch.randn(n, F, generator=g)
    cut = lambda t: [t[int(begin[r]):int(begin[r + 1])].contiguous() for r in range(P)]
    out = torch.cat(agg.forward(cut(X)))
    grad = torch.cat(agg.backward(cut(G)))
    A = torch.zeros(n, n, dtype=torch.float64)
    A.index_put_((d, s), torch.ones(s.numel(), dtype=torch.float64), accumulate=True)
    np.testing.assert_allclose(out.double().numpy(), (A @ X.double()).numpy(), rtol=0, atol=1e-4)
    np.testing.assert_allclose(grad.double().numpy(), (A.t() @ G.double()).numpy(), rtol=0, atol=1e-4)
    assert agg.edges_per_pass() == s.numel()
    assert sum(sum(p.recv_splits) for p in parts) == sum(sum(p.send_splits) for p in parts) > 0
