"""Numerical model behind the tensor-core dense kernels, in numpy (no GPU, no product code).

An fp32 product computed as three TF32 tensor-core products is limited not by the split (hi + lo
represents an fp32 value to 2^-22) but by the accumulator, which rounds toward zero once per MMA
instruction (8 products).  The kernels therefore keep the main product hi.hi and the two small
products in separate accumulators.  This test pins the error levels that choice rests on; the GPU
tests measure the same quantities on the hardware (tests/test_dense_gpu.py, bound 2e-6; measured
3.7e-7 with separate accumulators, 1.3e-6 with one)."""
import numpy as np


def _trunc_tf32(x):
    return (x.view(np.uint32) & np.uint32(0xFFFFE000)).view(np.float32)


def _rna_tf32(x):
    u = x.view(np.uint32).astype(np.uint64)
    return ((u + 0x1000) & 0xFFFFE000).astype(np.uint32).view(np.float32)


def _toward_zero(x64):
    f = x64.astype(np.float32)
    over = np.abs(f.astype(np.float64)) > np.abs(x64)
    f[over] = np.nextafter(f[over], np.float32(0))
    return f


def _accumulate(terms, K, rounding):
    acc = np.zeros((terms[0][0].shape[0], terms[0][1].shape[0]), np.float32)
    for k0 in range(0, K, 8):
        sl = slice(k0, k0 + 8)
        for x, y in terms:
            s = acc.astype(np.float64) + x[:, sl].astype(np.float64) @ y[:, sl].astype(np.float64).T
            acc = _toward_zero(s) if rounding == "rz" else s.astype(np.float32)
    return acc


def test_error_levels_of_the_three_product_scheme():
    rng = np.random.default_rng(0)
    M, N, K = 600, 48, 256
    a = rng.standard_normal((M, K)).astype(np.float32)
    w = rng.standard_normal((N, K)).astype(np.float32)
    a_hi = _trunc_tf32(a)                                  # the activation panel as the tensor core reads it
    a_lo = _rna_tf32((a - a_hi).astype(np.float32))
    w_hi = _rna_tf32(w)
    w_lo = _rna_tf32((w - w_hi).astype(np.float32))
    ref = a.astype(np.float64) @ w.astype(np.float64).T
    scale = np.abs(a).astype(np.float64) @ np.abs(w).astype(np.float64).T

    def err(c):
        return (np.abs(c.astype(np.float64) - ref) / scale).max()

    exact_sum = sum(x.astype(np.float64) @ y.astype(np.float64).T for x, y in ((a_hi, w_hi), (a_lo, w_hi), (a_hi, w_lo)))
    split_only = err(exact_sum)
    one_acc = err(_accumulate([(a_hi, w_lo), (a_hi, w_hi), (a_lo, w_hi)], K, "rz"))
    main = _accumulate([(a_hi, w_hi)], K, "rz")
    small = _accumulate([(a_hi, w_lo), (a_lo, w_hi)], K, "rz")
    two_acc = err(main + small)
    nearest = err(_accumulate([(a_hi, w_lo), (a_hi, w_hi), (a_lo, w_hi)], K, "rn"))
    fp32 = err(a @ w.T)
    assert split_only < 1e-7                 # the representation is not the limit
    assert 6e-7 < one_acc < 2e-6             # one truncating accumulator: what the first kernel measured
    assert two_acc < 0.6 * one_acc           # separate accumulators remove most full-magnitude roundings
    assert two_acc < 2.5 * fp32              # ... and land within a small factor of an fp32 product
    assert nearest < one_acc / 3             # the gap is the rounding mode, not the scheme
