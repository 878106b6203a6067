"""dropout -> LayerNorm -> ReLU between the layers as one fused forward and one fused backward
kernel (the reference runs F.dropout, LayerNorm and F.relu as separate passes,
self_benchmark/a64fx/model/DistSAGE.py:49-54).

`dropout_ln_relu(x, weight, bias, p, training, eps)` is the call; shapes the kernels do not take
(F not a multiple of 4 or above 1024, unaligned rows) fall back to the three torch ops.  The dropout
mask comes from a counter-based generator inside the kernel, keyed by a 64-bit seed drawn from
torch's CPU generator (so `torch.manual_seed` makes runs repeatable); it is not torch's mask.
"""
import warnings

import torch
import torch.nn.functional as F

from . import _lib

MODE = "fused"  # tests set "torch" to compare against the three separate ops

_partials = {}


def supported(x: torch.Tensor) -> bool:
    return (MODE == "fused" and x.is_cuda and x.dtype == torch.float32 and x.dim() == 2 and x.stride(1) == 1
            and x.size(1) % 4 == 0 and 0 < x.size(1) <= 1024 and x.stride(0) % 4 == 0 and x.data_ptr() % 16 == 0)


_warned = set()


def _torch_path(what: str, x: torch.Tensor) -> None:
    """Say once per width that a call went to the separate torch ops because the fused kernel does not
    take it (F not a multiple of 4 or above 1024, rows not 16-byte aligned)."""
    if MODE == "fused" and (what, x.size(-1)) not in _warned:
        _warned.add((what, x.size(-1)))
        warnings.warn(f"norm.{what}: width {x.size(-1)} / this row alignment is outside the fused kernel's range; "
                      "using the separate torch ops for it")


def _partial(device, f: int) -> torch.Tensor:
    key = (device.index, _lib.stream_ptr(device), f)
    buf = _partials.get(key)
    if buf is None:
        buf = torch.empty(_lib.lib().gnnagg_dropout_ln_relu_partial_bytes(f), dtype=torch.uint8, device=device)
        _partials[key] = buf
    return buf


class _DropoutLayerNormReLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, weight, bias, p, training, eps):
        rows, f = x.shape
        p = float(p) if training else 0.0
        need_grad = training and (x.requires_grad or weight.requires_grad or bias.requires_grad)
        y = torch.empty(rows, f, dtype=torch.float32, device=x.device)
        mask = torch.empty(rows * (f // 4), dtype=torch.uint8, device=x.device) if p > 0 else None
        stats = torch.empty(rows, 2, dtype=torch.float32, device=x.device) if need_grad else None
        seed = int(torch.empty((), dtype=torch.int64).random_()) if p > 0 else 0
        weight, bias = weight.contiguous(), bias.contiguous()
        rc = _lib.lib().gnnagg_dropout_ln_relu_fwd(x.data_ptr(), x.stride(0), rows, f, weight.data_ptr(), bias.data_ptr(),
                                                   float(eps), p, seed, y.data_ptr(), y.stride(0), _lib.ptr(mask),
                                                   _lib.ptr(stats), _lib.stream_ptr(x.device))
        _lib.check(rc, "dropout_ln_relu_fwd")
        if need_grad:
            ctx.save_for_backward(x, weight, bias, mask, stats)
            ctx.p = p
        return y

    @staticmethod
    def backward(ctx, gy):
        x, weight, bias, mask, stats = ctx.saved_tensors
        rows, f = x.shape
        if gy.stride(1) != 1 or gy.stride(0) % 4 != 0 or gy.data_ptr() % 16 != 0:
            gy = gy.contiguous()
        gx = torch.empty(rows, f, dtype=torch.float32, device=x.device)
        dgamma = torch.empty(f, dtype=torch.float32, device=x.device)
        dbeta = torch.empty(f, dtype=torch.float32, device=x.device)
        partial = _partial(x.device, f)
        rc = _lib.lib().gnnagg_dropout_ln_relu_bwd(gy.data_ptr(), gy.stride(0), x.data_ptr(), x.stride(0), _lib.ptr(mask),
                                                   stats.data_ptr(), weight.data_ptr(), bias.data_ptr(), rows, f, ctx.p,
                                                   gx.data_ptr(), gx.stride(0), partial.data_ptr(), partial.numel(),
                                                   dgamma.data_ptr(), dbeta.data_ptr(), _lib.stream_ptr(x.device))
        _lib.check(rc, "dropout_ln_relu_bwd")
        return gx, dgamma, dbeta, None, None, None


def dropout_ln_relu(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor, p: float, training: bool,
                    eps: float = 1e-5) -> torch.Tensor:
    """relu(layer_norm(dropout(x, p, training))) over the last dimension."""
    _lib.require_cuda(x, weight, bias)
    if supported(x) and weight is not None and bias is not None:
        return _DropoutLayerNormReLU.apply(x, weight, bias, p, training, eps)
    _torch_path("dropout_ln_relu", x)
    x = F.dropout(x, p=p, training=training)
    return F.relu(F.layer_norm(x, (x.size(-1),), weight, bias, eps))


class _ReluDropout_(torch.autograd.Function):
    """relu followed by dropout, in place on x, one pass each way."""

    @staticmethod
    def forward(ctx, x, p, training):
        rows, f = x.shape
        p = float(p) if training else 0.0
        need_grad = x.requires_grad
        mask = torch.empty(rows * (f // 4), dtype=torch.uint8, device=x.device) if need_grad else None
        seed = int(torch.empty((), dtype=torch.int64).random_()) if p > 0 else 0
        rc = _lib.lib().gnnagg_relu_dropout_fwd(x.data_ptr(), x.stride(0), rows, f, p, seed, x.data_ptr(), x.stride(0),
                                                _lib.ptr(mask), _lib.stream_ptr(x.device))
        _lib.check(rc, "relu_dropout_fwd")
        ctx.mark_dirty(x)
        ctx.p = p
        if need_grad:
            ctx.save_for_backward(mask)
        return x

    @staticmethod
    def backward(ctx, gy):
        (mask,) = ctx.saved_tensors
        if gy.stride(1) != 1 or gy.stride(0) % 4 != 0 or gy.data_ptr() % 16 != 0:
            gy = gy.contiguous()
        gx = torch.empty(gy.shape, dtype=torch.float32, device=gy.device)
        rc = _lib.lib().gnnagg_relu_dropout_bwd(gy.data_ptr(), gy.stride(0), mask.data_ptr(), gy.size(0), gy.size(1), ctx.p,
                                                gx.data_ptr(), gx.stride(0), _lib.stream_ptr(gy.device))
        _lib.check(rc, "relu_dropout_bwd")
        return gx, None, None


def relu_dropout_(x: torch.Tensor, p: float, training: bool) -> torch.Tensor:
    """dropout(relu(x)) written over x (x must not be needed by the backward of the op that made it)."""
    _lib.require_cuda(x)
    if supported(x):
        return _ReluDropout_.apply(x, p, training)
    _torch_path("relu_dropout_", x)
    x = F.relu(x, inplace=True)
    return F.dropout(x, p=p, training=training) if p > 0 else x
