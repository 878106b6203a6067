"""GNN layers and models that CALL the aggregation path (call sites, not the product).

DistSAGEConvGrad / DistSAGE keep the reference's structure and parameter names
(self_benchmark/a64fx/model/layers/sageconv.py:17-93, model/DistSAGE.py:14-69, model/utils.py:8-35)
so that its weights load key for key.  DistGCNConv / DistGCN are an addition: the reference has no
GCN layer; here GCN's symmetric normalisation is applied around the reference's aggregation op as
D^-1/2 (A+I) D^-1/2 X = d^-1/2 * Aggregate(d^-1/2 * X) on the unit-valued adjacency (self-loops are
edges of the graph), which works unchanged with pre/post-aggregation and the quantised halo.
"""
import random

import numpy as np
import torch
import torch.distributed as dist
import torch.nn.functional as F
from torch import Tensor
from torch.nn import LayerNorm, Linear, Parameter

from . import dense, norm
from .aggregator import Aggregator


class DistSAGEConvGrad(torch.nn.Module):
    def __init__(self, in_channels: int, out_channels: int, num_bits: int, is_pre_delay: bool,
                 add_self_loops: bool = False, normalize: bool = True, bias: bool = True, **kwargs):
        super().__init__()
        self.in_channels = in_channels
        self.out_channels = out_channels
        self.add_self_loops = add_self_loops
        self.normalize = normalize
        self.num_bits = num_bits
        self.is_pre_delay = is_pre_delay
        self.lin_neigh = Linear(in_channels, out_channels, bias=False)
        self.lin_self = Linear(in_channels, out_channels, bias=False)
        if bias:
            self.bias = Parameter(torch.zeros(out_channels))
        else:
            self.register_parameter("bias", None)

    def reset_parameters(self):
        gain = torch.nn.init.calculate_gain("relu")
        torch.nn.init.xavier_uniform_(self.lin_neigh.weight, gain=gain)
        torch.nn.init.xavier_uniform_(self.lin_self.weight, gain=gain)

    def propagate(self, graph, local_nodes_feat, layer):
        return Aggregator.apply(graph, local_nodes_feat, layer, self.num_bits, self.is_pre_delay, self.training)

    def forward(self, graph, local_nodes_feat, layer) -> Tensor:
        out = self.propagate(graph, local_nodes_feat, layer)
        if self.normalize:
            out = dense.RowDivide_.apply(out, graph.in_degrees)
        if dense.enabled():  # both products, the add and the bias in two tensor-core kernel calls
            return dense.SageDense.apply(out, local_nodes_feat, self.lin_neigh.weight, self.lin_self.weight, self.bias)
        out = self.lin_neigh(out)
        out += self.lin_self(local_nodes_feat)
        if self.bias is not None:
            out += self.bias
        return out


class DistSAGE(torch.nn.Module):
    def __init__(self, in_channels, hidden_channels, out_channels, num_layers=3, dropout=0.5, num_bits=32,
                 is_pre_delay=False):
        super().__init__()
        self.convs = torch.nn.ModuleList()
        self.norms = torch.nn.ModuleList()
        self.convs.append(DistSAGEConvGrad(in_channels, hidden_channels, num_bits, is_pre_delay))
        self.norms.append(LayerNorm(hidden_channels))
        for _ in range(num_layers - 2):
            self.convs.append(DistSAGEConvGrad(hidden_channels, hidden_channels, num_bits, is_pre_delay))
            self.norms.append(LayerNorm(hidden_channels))
        self.convs.append(DistSAGEConvGrad(hidden_channels, out_channels, num_bits, is_pre_delay))
        self.dropout = dropout

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()
        for norm in self.norms:
            norm.reset_parameters()

    def forward(self, graph, nodes_feats):
        for i, conv in enumerate(self.convs[:-1]):
            nodes_feats = conv(graph, nodes_feats, i)
            norm_i = self.norms[i]
            nodes_feats = norm.dropout_ln_relu(nodes_feats, norm_i.weight, norm_i.bias, self.dropout, self.training,
                                               norm_i.eps)
        nodes_feats = self.convs[-1](graph, nodes_feats, len(self.convs) - 1)
        return F.log_softmax(nodes_feats, dim=1)


class _ScaledAggregator(torch.autograd.Function):
    """d^-1/2 * Aggregate(d^-1/2 * x) as one autograd node: the two row scalings run in place on
    temporaries, so nothing but the degree vector is kept for backward (at 10^7 rows x 256 columns per
    GPU every saved activation is 14 GB)."""

    @staticmethod
    def forward(ctx, graph, x, dinv, layer, num_bits, is_pre_delay, is_training, bias=None):
        scaled = dense.scale_rows(x, dinv)
        out = Aggregator.forward(ctx, graph, scaled, layer, num_bits, is_pre_delay, is_training)
        del scaled
        dense.scale_rows(out, dinv, out=out, bias=bias)  # the layer's bias rides on the second scaling
        ctx.dinv = dinv
        ctx.has_bias = bias is not None
        return out

    @staticmethod
    def backward(ctx, grad_out):
        g = dense.scale_rows(grad_out if grad_out.stride(1) == 1 else grad_out.contiguous(), ctx.dinv)
        grad = Aggregator.backward(ctx, g)[1]
        del g
        dense.scale_rows(grad, ctx.dinv, out=grad)
        return None, grad, None, None, None, None, None, (grad_out.sum(0) if ctx.has_bias else None)


class DistGCNConv(torch.nn.Module):
    """out = d^-1/2 * Aggregate(d^-1/2 * h) + bias with h = x W when in_channels > out_channels
    (transform first, so the narrower tensor is aggregated and exchanged), else (d^-1/2 A d^-1/2 x) W."""

    def __init__(self, in_channels: int, out_channels: int, num_bits: int, is_pre_delay: bool, bias: bool = True):
        super().__init__()
        self.in_channels, self.out_channels = in_channels, out_channels
        self.num_bits, self.is_pre_delay = num_bits, is_pre_delay
        self.lin = Linear(in_channels, out_channels, bias=False)
        self.bias = Parameter(torch.zeros(out_channels)) if bias else None

    def reset_parameters(self):
        torch.nn.init.xavier_uniform_(self.lin.weight)
        if self.bias is not None:
            torch.nn.init.zeros_(self.bias)

    def forward(self, graph, x, layer) -> Tensor:
        dinv = graph.in_degrees.rsqrt()
        linear_first = self.in_channels > self.out_channels
        if dense.enabled():  # the bias goes into the epilogue of whichever kernel runs last
            if linear_first:
                h = dense.LinearTC.apply(x, self.lin.weight, None)
                return _ScaledAggregator.apply(graph, h, dinv, layer, self.num_bits, self.is_pre_delay, self.training,
                                               self.bias)
            h = _ScaledAggregator.apply(graph, x, dinv, layer, self.num_bits, self.is_pre_delay, self.training)
            return dense.LinearTC.apply(h, self.lin.weight, self.bias)
        h = self.lin(x) if linear_first else x
        h = _ScaledAggregator.apply(graph, h, dinv, layer, self.num_bits, self.is_pre_delay, self.training)
        if not linear_first:
            h = self.lin(h)
        if self.bias is not None:
            h += self.bias
        return h


class DistGCN(torch.nn.Module):
    def __init__(self, in_channels, hidden_channels, out_channels, num_layers=3, dropout=0.5, num_bits=32,
                 is_pre_delay=False):
        super().__init__()
        dims = [in_channels] + [hidden_channels] * (num_layers - 1) + [out_channels]
        self.convs = torch.nn.ModuleList(
            DistGCNConv(dims[i], dims[i + 1], num_bits, is_pre_delay) for i in range(num_layers))
        self.dropout = dropout

    def reset_parameters(self):
        for conv in self.convs:
            conv.reset_parameters()

    def forward(self, graph, x):
        for i, conv in enumerate(self.convs[:-1]):
            x = norm.relu_dropout_(conv(graph, x, i), self.dropout, self.training)
        return F.log_softmax(self.convs[-1](graph, x, len(self.convs) - 1), dim=1)


def create_model_and_optimizer(config: dict, device=None):
    """model/utils.py:8-29 of the reference: build, reset_parameters, DDP when world_size > 1, Adam.
    Weights are drawn on the CPU (so a seed gives the reference's initial weights) and then moved."""
    cls = {"sage": DistSAGE, "gcn": DistGCN}.get(config["model_name"])
    if cls is None:
        return None, None
    model = cls(config["in_channels"], config["hidden_channels"], config["out_channels"], config["num_layers"],
                config["dropout"], config["num_bits"], config["is_pre_delay"])
    model.reset_parameters()
    if device is not None:
        model = model.to(device)
    if dist.is_available() and dist.is_initialized() and dist.get_world_size() > 1:
        model = torch.nn.parallel.DistributedDataParallel(model)
    optimizer = torch.optim.Adam(model.parameters(), lr=config["lr"], weight_decay=config["weight_decay"])
    return model, optimizer


def set_random_seed(random_seed):
    torch.manual_seed(random_seed)
    np.random.seed(random_seed)
    random.seed(random_seed)
