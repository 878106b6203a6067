"""Fused dropout -> LayerNorm -> ReLU kernels against the three torch ops (fp64 reference)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _unpack_mask(mask_bytes, rows, f):
    bits = torch.stack([(mask_bytes >> i) & 1 for i in range(4)], dim=1)  # (rows*f/4, 4)
    return bits.reshape(rows, f).to(torch.float64)


def _reference(x, gamma, beta, keep, p, gy, eps=1e-5):
    xd = x.double().detach().requires_grad_(True)
    g = gamma.double().detach().requires_grad_(True)
    b = beta.double().detach().requires_grad_(True)
    d = xd * keep / (1.0 - p) if keep is not None else xd
    y = F.relu(F.layer_norm(d, (x.size(1),), g, b, eps))
    y.backward(gy.double())
    return y.detach(), xd.grad, g.grad, b.grad


@pytest.mark.parametrize("rows,f", [(1000, 256), (1, 128), (777, 100), (513, 172), (300, 512), (65, 1024), (4099, 4)])
@pytest.mark.parametrize("p", [0.0, 0.5])
def test_fused_matches_torch(rows, f, p):
    from gnn_benchmark_b200 import norm

    g = torch.Generator(device="cuda").manual_seed(rows + f)
    x = torch.randn(rows, f, device="cuda", generator=g, requires_grad=True)
    gamma = (torch.rand(f, device="cuda", generator=g) + 0.5).requires_grad_(True)
    beta = (torch.randn(f, device="cuda", generator=g) * 0.1).requires_grad_(True)
    gy = torch.randn(rows, f, device="cuda", generator=g)
    assert norm.supported(x)
    torch.manual_seed(7)
    y = norm.dropout_ln_relu(x, gamma, beta, p, True)
    saved = y.grad_fn.saved_tensors
    keep = None
    if p > 0:
        keep = _unpack_mask(saved[3], rows, f)
        if rows * f > 20000:
            assert abs(keep.mean().item() - (1 - p)) < 0.02
    y.backward(gy)
    p_eff = round(p * 65536) / 65536
    ry, rgx, rgg, rgb = _reference(x, gamma, beta, keep, p_eff, gy)
    torch.testing.assert_close(y.double(), ry, rtol=1e-5, atol=2e-5)
    # rows whose ReLU decision sits within rounding of zero may differ between fp32 and fp64
    torch.testing.assert_close(x.grad.double(), rgx, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(gamma.grad.double(), rgg, rtol=1e-4, atol=1e-3 * max(1.0, rows ** 0.5 / 10))
    torch.testing.assert_close(beta.grad.double(), rgb, rtol=1e-4, atol=1e-3 * max(1.0, rows ** 0.5 / 10))


def test_mask_is_seeded_and_changes():
    from gnn_benchmark_b200 import norm

    x = torch.randn(512, 256, device="cuda", requires_grad=True)
    w = torch.ones(256, device="cuda")
    b = torch.zeros(256, device="cuda")
    torch.manual_seed(1)
    a1 = norm.dropout_ln_relu(x, w, b, 0.5, True)
    a2 = norm.dropout_ln_relu(x, w, b, 0.5, True)
    torch.manual_seed(1)
    b1 = norm.dropout_ln_relu(x, w, b, 0.5, True)
    assert torch.equal(a1, b1) and not torch.equal(a1, a2)


def test_eval_mode_has_no_dropout_and_keeps_nothing():
    from gnn_benchmark_b200 import norm

    x = torch.randn(300, 256, device="cuda")
    w = torch.rand(256, device="cuda") + 0.5
    b = torch.randn(256, device="cuda")
    y = norm.dropout_ln_relu(x, w, b, 0.5, False)
    ref = F.relu(F.layer_norm(x, (256,), w, b))
    torch.testing.assert_close(y, ref, rtol=1e-5, atol=1e-5)
    assert y.grad_fn is None


def test_unsupported_shapes_fall_back():
    from gnn_benchmark_b200 import norm

    x = torch.randn(64, 50, device="cuda")  # 50 % 4 != 0
    assert not norm.supported(x)
    w, b = torch.ones(50, device="cuda"), torch.zeros(50, device="cuda")
    y = norm.dropout_ln_relu(x, w, b, 0.0, True)
    torch.testing.assert_close(y, F.relu(F.layer_norm(x, (50,), w, b)))


@pytest.mark.parametrize("p", [0.0, 0.5])
def test_relu_dropout_inplace(p):
    from gnn_benchmark_b200 import norm

    g = torch.Generator(device="cuda").manual_seed(3)
    base = torch.randn(2000, 172, device="cuda", generator=g, requires_grad=True)
    x = base * 1.0
    x0 = x.detach().clone()
    torch.manual_seed(11)
    y = norm.relu_dropout_(x, p, True)
    assert y.data_ptr() == x.data_ptr()
    keep = _unpack_mask(y.grad_fn.saved_tensors[0], 2000, 172).float()
    scale = 1.0 / (1.0 - round(p * 65536) / 65536)
    assert torch.equal(keep, keep * (x0 > 0))  # a passed gradient implies a positive input
    torch.testing.assert_close(y.detach(), torch.relu(x0) * keep * scale + 0.0 * x0, rtol=1e-6, atol=0)
    if p > 0:
        frac = (keep.sum() / (x0 > 0).sum()).item()
        assert abs(frac - (1 - p)) < 0.02
    else:
        assert torch.equal(keep, (x0 > 0).float())
    gy = torch.randn(2000, 172, device="cuda", generator=g)
    y.backward(gy)
    torch.testing.assert_close(base.grad, gy * keep * scale, rtol=1e-6, atol=0)


def test_keep_bits_match_philox_restatement():
    """Bit-exact: the kernels' dropout decisions against the numpy Philox-4x32-10 restatement
    (tests/util.py, pinned to the generator's published known-answer vectors)."""
    import numpy as np

    from gnn_benchmark_b200 import norm
    from util import dropout_keep_bits

    rows, f = 300, 256
    x = torch.randn(rows, f, device="cuda", requires_grad=True)
    w, b = torch.ones(f, device="cuda"), torch.zeros(f, device="cuda")
    for p in (0.5, 0.1):
        torch.manual_seed(7)
        y = norm.dropout_ln_relu(x, w, b, p, True)
        got = y.grad_fn.saved_tensors[3].cpu().numpy().reshape(rows, f // 4)
        torch.manual_seed(7)
        seed = int(torch.empty((), dtype=torch.int64).random_())
        assert np.array_equal(got, dropout_keep_bits(rows, f // 4, seed, p))
    h = (x * 1.0)
    positive = (h.detach() > 0).cpu().numpy().reshape(rows, f // 4, 4)
    pos_bits = (positive * np.array([1, 2, 4, 8])).sum(-1).astype(np.uint8)
    torch.manual_seed(9)
    z = norm.relu_dropout_(h, 0.5, True)
    got = z.grad_fn.saved_tensors[0].cpu().numpy().reshape(rows, f // 4)
    torch.manual_seed(9)
    seed = int(torch.empty((), dtype=torch.int64).random_())
    assert np.array_equal(got, dropout_keep_bits(rows, f // 4, seed, 0.5) & pos_bits)
