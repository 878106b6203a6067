"""The added GCN layer: d^-1/2 (A+I) d^-1/2 X W through the aggregation op equals the dense
normalised-adjacency product, forward and gradients, on one rank and on four emulated ranks (forward)."""
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def test_gcn_conv_matches_dense_normalised_adjacency(cuda_lib):
    from gnn_benchmark_b200 import Communicator, Quantizer_for_all_procs, TimeRecorder, graphgen
    from gnn_benchmark_b200.data_manager.DataLoader import build_graph
    from gnn_benchmark_b200.model import DistGCNConv

    n = 500
    src, dst = graphgen.erdos_renyi_edges(n, 3000, seed=5, device="cuda")
    src, dst = graphgen.symmetrize(src, dst, n, self_loops=True)
    begin = graphgen.contiguous_partitions(n, 1)
    Communicator(32)
    Quantizer_for_all_procs(1, 32)
    TimeRecorder(1, 1)
    local, remote = graphgen.partition_edges(src, dst, begin, 0)
    for cin, cout in ((24, 40), (40, 8)):  # aggregate-first and transform-first
        graph = build_graph(local, remote, begin, 0, 1, max(cin, cout), 32, False, device="cuda")
        torch.manual_seed(0)
        conv = DistGCNConv(cin, cout, 32, False).cuda()
        conv.reset_parameters()
        x = torch.randn(n, cin, device="cuda", requires_grad=True)
        out = conv(graph, x, 0)
        g = torch.randn_like(out)
        out.backward(g)
        A = torch.zeros(n, n, device="cuda", dtype=torch.float64)
        A[dst, src] = 1.0
        d = A.sum(1)
        An = A / torch.sqrt(d)[:, None] / torch.sqrt(d)[None, :]
        xd = x.detach().double().requires_grad_()
        W = conv.lin.weight.detach().double()
        ref = An @ xd @ W.t() + conv.bias.detach().double()
        ref.backward(g.double())
        assert torch.allclose(out.double(), ref, rtol=1e-5, atol=1e-5)
        assert torch.allclose(x.grad.double(), xd.grad, rtol=1e-5, atol=1e-5)
