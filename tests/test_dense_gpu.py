"""Tensor-core dense transform (gnnagg_dense_tf32x3_f32) against an fp64 product.

Tolerance: |C - C64| <= 2e-6 * (|A| |B|^T) element-wise.  A single-pass TF32 product misses this by
two orders of magnitude (2^-11 per operand), fp32 FMA chains sit near 1e-7 * sqrt(K)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(M, N, K, bias, accumulate, lda_pad=0, ldc_pad=0, seed=0):
    from gnn_benchmark_b200 import dense

    g = torch.Generator(device="cuda").manual_seed(seed)
    a_full = torch.randn(M, K + lda_pad, device="cuda", generator=g)
    a = a_full[:, :K]
    w = torch.randn(N, K, device="cuda", generator=g)
    b = torch.randn(N, device="cuda", generator=g) if bias else None
    c_full = torch.randn(M, N + ldc_pad, device="cuda", generator=g)
    c = c_full[:, :N]
    ref = a.double() @ w.double().t()
    if bias:
        ref += b.double()
    if accumulate:
        ref += c.double()
    scale = a.abs().double() @ w.abs().double().t() + (c.abs().double() if accumulate else 0) + 1e-30
    guard = c_full[:, N:].clone()
    dense.linear(a, w, b, out=c, accumulate=accumulate)
    dense.check_status()
    err = ((c.double() - ref).abs() / scale).max().item()
    assert err <= 2e-6, f"M={M} N={N} K={K}: relative error {err:.3e}"
    assert torch.equal(c_full[:, N:], guard), "wrote outside the N output columns"


@pytest.mark.parametrize("M,N,K", [
    (128, 16, 32), (256, 64, 64), (1000, 256, 256), (128 * 148 * 2 + 77, 256, 100), (5000, 47, 256),
    (3001, 100, 256), (4096, 172, 256), (70, 16, 8), (1, 256, 128), (129, 48, 36), (777, 128, 512),
])
def test_dense_matches_fp64(M, N, K):
    _case(M, N, K, bias=False, accumulate=False)


@pytest.mark.parametrize("bias,accumulate", [(True, False), (False, True), (True, True)])
def test_dense_bias_and_accumulate(bias, accumulate):
    _case(2500, 256, 256, bias, accumulate, seed=1)
    _case(999, 47, 100, bias, accumulate, seed=2)


def test_dense_strided_operands():
    _case(1500, 172, 128, bias=True, accumulate=True, lda_pad=4, ldc_pad=3, seed=3)


def test_dense_special_values():
    """NaN inputs give NaN rows, zero rows give exact zeros, rows with an infinity come out non-finite
    (the split sends +inf through products of both signs, so some columns read NaN where an fp32 FMA
    chain reads +-inf); all other rows are untouched by their neighbours."""
    from gnn_benchmark_b200 import dense

    a = torch.randn(256, 64, device="cuda")
    w = torch.randn(32, 64, device="cuda")
    a[3, 5] = float("inf")
    a[7, 0] = float("nan")
    a[9] = 0
    c = dense.linear(a, w)
    dense.check_status()
    ref = a.double() @ w.double().t()
    assert torch.isnan(c[7]).all()
    assert not torch.isfinite(c[3]).any()
    assert torch.equal(c[9], torch.zeros_like(c[9]))
    rest = [i for i in range(256) if i not in (3, 7)]
    assert torch.isfinite(c[rest]).all()
    torch.testing.assert_close(c[rest].double(), ref[rest], rtol=1e-5, atol=1e-4)


def test_scale_rows_matches_torch():
    from gnn_benchmark_b200 import dense

    x = torch.randn(1001, 172, device="cuda")
    s = torch.rand(1001, 1, device="cuda") + 0.5
    assert torch.equal(dense.scale_rows(x, s, divide=True), x / s)
    assert torch.equal(dense.scale_rows(x, s), x * s)
    y = x.clone()
    dense.scale_rows(y, s, out=y)
    assert torch.equal(y, x * s)
    b = torch.randn(172, device="cuda")
    assert torch.equal(dense.scale_rows(x, s, bias=b), x * s + b)
    x2 = torch.randn(77, 47, device="cuda", requires_grad=True)  # scalar path, through autograd
    s2 = torch.rand(77, 1, device="cuda") + 1.0
    out = dense.RowDivide_.apply(x2 * 1.0, s2)
    out.backward(torch.ones_like(out))
    assert torch.equal(out.detach(), (x2 / s2).detach()) and torch.equal(x2.grad, (1.0 / s2).expand(77, 47))


def test_dense_rejects_unsupported():
    from gnn_benchmark_b200 import dense

    a = torch.randn(64, 47, device="cuda")  # 188-byte rows: not TMA-addressable
    w = torch.randn(16, 47, device="cuda")
    assert not dense.supported(a, 16)
    with pytest.raises(RuntimeError):
        dense.linear(a, w)
    assert not dense.supported(torch.randn(64, 64, device="cuda"), 300)


@pytest.mark.parametrize("k_in,n_out", [(100, 256), (256, 47)])
def test_sage_dense_autograd_matches_torch(k_in, n_out):
    """Forward and all five gradients of the layer's dense half; n_out = 47 exercises the zero-padded
    upstream gradient (rows of 47 floats are not TMA-addressable)."""
    from gnn_benchmark_b200 import dense

    old = dense.MODE
    dense.MODE = "tf32x3"
    try:
        g = torch.Generator(device="cuda").manual_seed(5)
        aggr = torch.randn(3000, k_in, device="cuda", generator=g, requires_grad=True)
        x = torch.randn(3000, k_in, device="cuda", generator=g, requires_grad=True)
        wn = torch.randn(n_out, k_in, device="cuda", generator=g, requires_grad=True)
        ws = torch.randn(n_out, k_in, device="cuda", generator=g, requires_grad=True)
        b = torch.randn(n_out, device="cuda", generator=g, requires_grad=True)
        go = torch.randn(3000, n_out, device="cuda", generator=g)
        out = dense.SageDense.apply(aggr, x, wn, ws, b)
        out.backward(go)
        got = [out.detach()] + [t.grad.clone() for t in (aggr, x, wn, ws, b)]
        for t in (aggr, x, wn, ws, b):
            t.grad = None
        ref = aggr.double() @ wn.double().t() + x.double() @ ws.double().t() + b.double()
        ref.backward(go.double())
        want = [ref.detach()] + [t.grad for t in (aggr, x, wn, ws, b)]
        dense.check_status()
        for a_, b_ in zip(got, want):
            torch.testing.assert_close(a_.double(), b_.double(), rtol=1e-5, atol=1e-3)
    finally:
        dense.MODE = old


@pytest.mark.parametrize("M,N,K", [
    (16, 32, 32), (1000, 256, 256), (40000, 256, 100), (5000, 128, 256), (3333, 172, 256), (777, 100, 48),
    (200000, 256, 256), (15, 256, 128), (700000, 64, 96), (148 * 2048 + 16, 172, 32),
])
def test_wgrad_matches_fp64(M, N, K):
    """dW = G^T X against fp64; same element-wise bound as the forward product.  The last two shapes
    give every CTA more than 2048 rows, so the periodic move of the accumulator to scratch runs."""
    from gnn_benchmark_b200 import dense

    g = torch.Generator(device="cuda").manual_seed(M + N)
    G = torch.randn(M, N, device="cuda", generator=g)
    X = torch.randn(M, K, device="cuda", generator=g)
    out = dense.wgrad(G, X)
    dense.check_status()
    ref = G.double().t() @ X.double()
    scale = G.abs().double().t() @ X.abs().double() + 1e-30
    err = ((out.double() - ref).abs() / scale).max().item()
    assert err <= 2e-6, f"M={M} N={N} K={K}: relative error {err:.3e}"


def test_wgrad_rejects_unsupported():
    from gnn_benchmark_b200 import dense

    g = torch.randn(64, 47, device="cuda")
    x = torch.randn(64, 64, device="cuda")
    assert not dense.wgrad_supported(g, x)
    with pytest.raises(RuntimeError):
        dense.wgrad(g, x)


def test_bounded_waits_give_up_and_report():
    """The give-up path of the tensor-core kernels: with the stall hook on, a launch announces 16 bytes
    more to its load barriers than its copies deliver, so the first wait for a load runs out (3 ms limit
    here, one second in normal operation).  The kernel must return by itself with the code of that wait
    in its status word (2: a consumer of the loaded tile; 5: the epilogue warps, whose wait for the
    accumulator starts at the same moment and may run out first), and the next normal launches on the
    same device, same workspaces included, must be correct."""
    from gnn_benchmark_b200 import _lib, dense

    lib = _lib.lib()
    g = torch.Generator(device="cuda").manual_seed(11)
    a = torch.randn(256, 64, device="cuda", generator=g)
    w = torch.randn(16, 64, device="cuda", generator=g)
    gr = torch.randn(256, 16, device="cuda", generator=g)
    dense.linear(a, w)          # workspaces exist and are clean before the hook goes on
    dense.wgrad(gr, a)
    dense.check_status()
    for call, codes in ((lambda: dense.linear(a, w), (2, 5)), (lambda: dense.wgrad(gr, a), (2,))):
        _lib.check(lib.gnnagg_dense_stall_test(16, 3000), "stall_test")
        try:
            call()
            torch.cuda.synchronize()   # the kernel returned: nothing hangs, no CUDA error
        finally:
            _lib.check(lib.gnnagg_dense_stall_test(0, 0), "stall_test")
        with pytest.raises(RuntimeError, match=r"reported status (\d)") as info:
            dense.check_status()
        assert int(info.value.args[0].split("reported status ")[1][0]) in codes
        dense.clear_status()
        dense.check_status()
    # the same shapes (same workspaces) and a full-size one, after the give-ups
    out = dense.linear(a, w)
    ref = a.double() @ w.double().t()
    scale = a.abs().double() @ w.abs().double().t()
    assert ((out.double() - ref).abs() / scale).max().item() <= 2e-6
    dw = dense.wgrad(gr, a)
    ref = gr.double().t() @ a.double()
    scale = gr.abs().double().t() @ a.abs().double()
    assert ((dw.double() - ref).abs() / scale).max().item() <= 2e-6
    _case(1000, 256, 256, bias=True, accumulate=False, seed=5)
    assert lib.gnnagg_dense_stall_test(-1, 0) != 0 and lib.gnnagg_dense_stall_test(16, 10**7) != 0
