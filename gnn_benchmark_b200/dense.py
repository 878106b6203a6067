"""Dense feature transforms either side of the aggregation, on the tensor cores.

The reference's layer computes lin_neigh(aggr / deg) + lin_self(x) + bias with two fp32 nn.Linear
calls and two in-place adds (self_benchmark/a64fx/model/layers/sageconv.py:82-91).  Here the same
arithmetic goes through `gnnagg_dense_tf32x3_f32`: a tcgen05 GEMM that keeps fp32-grade accuracy by
splitting every operand into two TF32 pieces (three tensor-core products per fp32 product), with
the bias and the second product accumulated in the kernel's epilogue.

`linear(x, weight, bias, out, accumulate)` is the plain call; `SageDense` and `LinearTC` are the
autograd nodes the models use; `wgrad(g, x)` is the weight gradient G^T X (a reduction over all rows
into a small matrix) on the same tensor-core scheme.  Shapes the kernels do not take (more than 256
output columns, operand rows not 16-byte aligned) go to cuBLAS: `supported()` / `wgrad_supported()`
say which.
"""
import warnings

import torch

from . import _lib

MAX_N = 256
# "tf32x3": the tensor-core kernels wherever `supported()`.  Tests and the epoch benchmark set
# "cublas" (torch's fp32 matmul) to have the library call the kernels replace measured beside them.
MODE = "tf32x3"

_workspaces = {}


def enabled() -> bool:
    return MODE == "tf32x3"


_warned = set()


def _library_path(what: str, shape) -> None:
    """Say once per shape that a product went to cuBLAS because the tensor-core kernel does not take it."""
    key = (what, tuple(shape))
    if enabled() and key not in _warned:
        _warned.add(key)
        warnings.warn(f"dense.{what}: shape {tuple(shape)} is outside the tensor-core kernel's range "
                      f"(at most {MAX_N} output columns, 16-byte aligned operand rows); using torch.matmul for it")


def supported(a: torch.Tensor, n_out: int) -> bool:
    """Can `a` (M x K fp32) be the left operand of the tensor-core kernel with n_out output columns?"""
    return (a.is_cuda and a.dtype == torch.float32 and a.dim() == 2 and a.size(1) > 0 and a.stride(1) == 1
            and a.stride(0) % 4 == 0 and a.data_ptr() % 16 == 0 and 0 < n_out <= MAX_N
            and a.size(0) < 2 ** 31 - 128)


def _workspace(device: torch.device, n: int, k: int) -> torch.Tensor:
    key = (device.index, _lib.stream_ptr(device), n, k)
    ws = _workspaces.get(key)
    if ws is None:
        nbytes = _lib.lib().gnnagg_dense_workspace_bytes(n, k)
        ws = torch.zeros(nbytes, dtype=torch.uint8, device=device)  # zeroed: the status word starts at 0
        _workspaces[key] = ws
    return ws


def linear(x: torch.Tensor, weight: torch.Tensor, bias: torch.Tensor = None, out: torch.Tensor = None,
           accumulate: bool = False) -> torch.Tensor:
    """out (+)= x @ weight.T (+ bias) through the C ABI.  x (M,K), weight (N,K), out (M,N), all fp32."""
    _lib.require_cuda(x, weight, bias, out)
    if x.dim() != 2 or weight.dim() != 2 or x.size(1) != weight.size(1):
        raise RuntimeError(f"dense.linear: shape mismatch x={tuple(x.shape)} weight={tuple(weight.shape)}")
    if x.dtype != torch.float32 or weight.dtype != torch.float32:
        raise RuntimeError("dense.linear: operands must be float32")
    M, K = x.shape
    N = weight.size(0)
    if out is None:
        if accumulate:
            raise RuntimeError("dense.linear: accumulate needs an output to accumulate into")
        out = torch.empty(M, N, dtype=torch.float32, device=x.device)
    if out.shape != (M, N) or out.dtype != torch.float32 or out.stride(1) != 1:
        raise RuntimeError("dense.linear: out must be (M,N) float32 with unit inner stride")
    if not supported(x, N):
        raise RuntimeError("dense.linear: operand not supported by the tensor-core kernel (see supported())")
    if weight.stride(1) != 1:
        weight = weight.contiguous()
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != N or not bias.is_contiguous()):
        raise RuntimeError("dense.linear: bias must be a contiguous float32 vector of N elements")
    if M == 0:
        return out
    ws = _workspace(x.device, N, K)
    rc = _lib.lib().gnnagg_dense_tf32x3_f32(x.data_ptr(), x.stride(0), weight.data_ptr(), weight.stride(0),
                                            out.data_ptr(), out.stride(0), M, N, K, _lib.ptr(bias),
                                            1 if accumulate else 0, ws.data_ptr(), ws.numel(),
                                            _lib.stream_ptr(x.device))
    _lib.check(rc, "dense_tf32x3_f32")
    return out


def wgrad_supported(g: torch.Tensor, x: torch.Tensor) -> bool:
    def ok(t):
        return (t.is_cuda and t.dtype == torch.float32 and t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 4 == 0
                and t.data_ptr() % 16 == 0 and 0 < t.size(1) <= MAX_N)
    return ok(g) and ok(x) and g.size(0) == x.size(0) and g.size(0) < 2 ** 31 - 128


def wgrad(g: torch.Tensor, x: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """out = g.T @ x through the C ABI: g (M,N), x (M,K) -> (N,K), the gradient of a Linear weight."""
    _lib.require_cuda(g, x, out)
    if not wgrad_supported(g, x):
        raise RuntimeError("dense.wgrad: operands not supported by the tensor-core kernel (see wgrad_supported())")
    M, N = g.shape
    K = x.size(1)
    if out is None:
        out = torch.empty(N, K, dtype=torch.float32, device=g.device)
    if out.shape != (N, K) or out.dtype != torch.float32 or out.stride(1) != 1:
        raise RuntimeError("dense.wgrad: out must be (N,K) float32 with unit inner stride")
    key = (g.device.index, _lib.stream_ptr(g.device), "w", N, K)
    ws = _workspaces.get(key)
    if ws is None:
        ws = torch.zeros(_lib.lib().gnnagg_dense_wgrad_workspace_bytes(N, K), dtype=torch.uint8, device=g.device)
        _workspaces[key] = ws
    rc = _lib.lib().gnnagg_dense_wgrad_tf32x3_f32(g.data_ptr(), g.stride(0), x.data_ptr(), x.stride(0), M, N, K,
                                                  out.data_ptr(), out.stride(0), ws.data_ptr(), ws.numel(),
                                                  _lib.stream_ptr(g.device))
    _lib.check(rc, "dense_wgrad_tf32x3_f32")
    return out


def _matmul_tn(g: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
    """g.T @ x, tensor-core kernel when it takes the shapes, cuBLAS otherwise."""
    if enabled() and wgrad_supported(g, x):
        return wgrad(g, x)
    _library_path("wgrad", (g.size(1), x.size(1)))
    return g.t() @ x


def check_status(device=None) -> None:
    """Synchronise and raise if any dense kernel on `device` gave up on a wait (diagnostic)."""
    for key, ws in list(_workspaces.items()):
        dev, n, k = key[0], key[-2], key[-1]
        if device is not None and torch.device(device).index not in (None, dev):
            continue
        code = _lib.lib().gnnagg_dense_status(ws.data_ptr(), _lib.stream_ptr(ws.device))
        if code != 0:
            raise RuntimeError(f"dense kernel (N={n}, K={k}) reported status {code}: "
                               + ("a bounded wait inside the kernel ran out" if code > 0 else
                                  _lib.lib().gnnagg_error_string(code).decode()))


def clear_status(device=None) -> None:
    """Reset the status words check_status reads (after a reported time-out has been handled)."""
    for key, ws in list(_workspaces.items()):
        if device is not None and torch.device(device).index not in (None, key[0]):
            continue
        _lib.check(_lib.lib().gnnagg_dense_status_clear(ws.data_ptr(), _lib.stream_ptr(ws.device)), "dense_status_clear")


def scale_rows(x: torch.Tensor, s: torch.Tensor, divide: bool = False, out: torch.Tensor = None,
               bias: torch.Tensor = None) -> torch.Tensor:
    """out[i,:] = x[i,:] * s[i] (or / s[i]) (+ bias); s has one element per row; out=x scales in place."""
    _lib.require_cuda(x, s, out, bias)
    if bias is not None and (bias.dtype != torch.float32 or bias.numel() != x.size(1) or not bias.is_contiguous()):
        raise RuntimeError("scale_rows: bias must be a contiguous float32 vector with one element per column")
    if x.dim() != 2 or x.dtype != torch.float32 or x.stride(1) != 1 or s.dtype != torch.float32 \
            or s.numel() != x.size(0) or not s.is_contiguous():
        raise RuntimeError("scale_rows: x must be (rows,F) float32 with unit inner stride, s float32 with rows elements")
    if out is None:
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
    if out.shape != x.shape or out.dtype != torch.float32 or out.stride(1) != 1:
        raise RuntimeError("scale_rows: out must match x")
    rc = _lib.lib().gnnagg_scale_rows_f32(x.data_ptr(), x.stride(0), s.data_ptr(), x.size(0), x.size(1),
                                          1 if divide else 0, _lib.ptr(bias), out.data_ptr(), out.stride(0),
                                          _lib.stream_ptr(x.device))
    _lib.check(rc, "scale_rows_f32")
    return out


class RowDivide_(torch.autograd.Function):
    """x /= s row-wise, in place (the layer's `out /= graph.in_degrees`); gradient g / s."""

    @staticmethod
    def forward(ctx, x, s):
        ctx.s = s
        ctx.mark_dirty(x)
        return scale_rows(x, s, True, out=x)

    @staticmethod
    def backward(ctx, g):
        g = g if g.stride(1) == 1 else g.contiguous()
        return scale_rows(g, ctx.s, True), None


def _matmul_nt(a: torch.Tensor, w: torch.Tensor, bias=None, out=None, accumulate=False) -> torch.Tensor:
    """a @ w.T (+bias), tensor-core kernel when it takes the shape, cuBLAS otherwise."""
    if enabled() and supported(a, w.size(0)):
        return linear(a, w, bias, out, accumulate)
    _library_path("linear", (w.size(0), a.size(1)))
    r = a @ w.t()
    if bias is not None:
        r += bias
    if out is None:
        return r
    if accumulate:
        out += r
    else:
        out.copy_(r)
    return out


def _tma_rows(g: torch.Tensor) -> torch.Tensor:
    """`g` itself when its rows are 16-byte addressable, else a copy whose rows are padded with zero
    columns to a multiple of 4 (an upstream gradient of 47 columns has 188-byte rows, which TMA cannot
    address; the extra columns meet zero rows of the weight / are dropped from the weight gradient)."""
    if not enabled() or not g.is_cuda or g.dim() != 2 or g.size(1) % 4 == 0 or g.size(1) > MAX_N - 3:
        return g
    pad = torch.zeros(g.size(0), (g.size(1) + 3) // 4 * 4, dtype=g.dtype, device=g.device)
    pad[:, :g.size(1)] = g
    return pad


def _input_grad(g: torch.Tensor, weight: torch.Tensor) -> torch.Tensor:
    """g @ weight for an upstream gradient g (M,N) (possibly column-padded) and a Linear weight (N,K)."""
    wt = weight.t()
    if g.size(1) != weight.size(0):  # padded gradient: pad the transposed weight with zero columns
        wt_p = torch.zeros(weight.size(1), g.size(1), dtype=weight.dtype, device=weight.device)
        wt_p[:, :weight.size(0)] = wt
        return _matmul_nt(g, wt_p)
    return _matmul_nt(g, wt.contiguous())


def _weight_grad(g: torch.Tensor, x: torch.Tensor, n_out: int) -> torch.Tensor:
    """g^T @ x, dropping the rows that belong to padding columns of g."""
    gw = _matmul_tn(g, x)
    return gw if gw.size(0) == n_out else gw[:n_out].contiguous()


class LinearTC(torch.autograd.Function):
    """y = x @ W^T (+ b) with the forward and the input gradient on the tensor-core kernel."""

    @staticmethod
    def forward(ctx, x, weight, bias):
        ctx.save_for_backward(x, weight)
        ctx.has_bias = bias is not None
        return _matmul_nt(x, weight, bias)

    @staticmethod
    def backward(ctx, g):
        x, weight = ctx.saved_tensors
        g = g.contiguous()
        gx = gw = gb = None
        if ctx.has_bias and ctx.needs_input_grad[2]:
            gb = g.sum(0)
        g = _tma_rows(g)
        if ctx.needs_input_grad[0]:
            gx = _input_grad(g, weight)
        if ctx.needs_input_grad[1]:
            gw = _weight_grad(g, x, weight.size(0))
        return gx, gw, gb


class SageDense(torch.autograd.Function):
    """out = aggr @ Wn^T + x @ Ws^T (+ b): the dense half of a GraphSAGE layer as one node (the second
    product and the bias are accumulated by the kernel's epilogue instead of separate passes)."""

    @staticmethod
    def forward(ctx, aggr, x, w_neigh, w_self, bias):
        ctx.save_for_backward(aggr, x, w_neigh, w_self)
        ctx.has_bias = bias is not None
        out = torch.empty(aggr.size(0), w_neigh.size(0), dtype=torch.float32, device=aggr.device)
        _matmul_nt(aggr, w_neigh, None, out, False)
        _matmul_nt(x, w_self, bias, out, True)
        return out

    @staticmethod
    def backward(ctx, g):
        aggr, x, w_neigh, w_self = ctx.saved_tensors
        g = g.contiguous()
        g_aggr = g_x = g_wn = g_ws = g_b = None
        if ctx.has_bias and ctx.needs_input_grad[4]:
            g_b = g.sum(0)
        g = _tma_rows(g)
        n_out = w_neigh.size(0)
        if ctx.needs_input_grad[0]:
            g_aggr = _input_grad(g, w_neigh)
        if ctx.needs_input_grad[1]:
            g_x = _input_grad(g, w_self)
        if ctx.needs_input_grad[2]:
            g_wn = _weight_grad(g, aggr, n_out)
        if ctx.needs_input_grad[3]:
            g_ws = _weight_grad(g, x, n_out)
        return g_aggr, g_x, g_wn, g_ws, g_b
