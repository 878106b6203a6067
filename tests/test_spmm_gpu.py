"""K1 parity: the CUDA SpMM (through the C ABI) against the CPU oracle of the reference's
spmm (oracle/gnnagg_oracle.c), the committed output of the compiled reference, and
size-independent properties at the benchmark's full size.

Tolerance (north_star): SpMM outputs within 1e-5 relative -- fp32 summation-order differences
only; rows handled by one chunk at F > 64 are bit-identical to the reference order."""
import os

import numpy as np
import pytest
import torch

import oracle
from util import random_csr, rel_err, to_dev

pytestmark = pytest.mark.gpu

RTOL = 1e-5
ATOL = 1e-5


def assert_spmm_close(got, want, rowptr, col, val, X, out0=None, rtol=RTOL):
    """|got - want| <= rtol * (|out0| + |A| |X|) element-wise: 1e-5 relative to the magnitude of the
    terms summed, the yardstick under which two fp32 summation orders of the same row agree
    (a cancelling sum has no meaningful error relative to its own tiny value)."""
    scale = oracle.spmm(rowptr, col, np.abs(val), np.abs(X), None if out0 is None else np.abs(out0).copy())
    err = np.abs(got.astype(np.float64) - want.astype(np.float64))
    bad = err > rtol * scale + 1e-30
    assert not bad.any(), f"{bad.sum()} elements off; worst ratio {np.max(err / (scale + 1e-30)):.3e}"


def run_spmm(cuda_lib, rowptr, col, val, K, X, out0=None, accumulate=True):
    from gnn_benchmark_b200 import spmm_kernel

    rp, c, v = to_dev(rowptr, torch.int64), to_dev(col, torch.int32), to_dev(val, torch.float32)
    Xd = to_dev(X)
    M = len(rowptr) - 1
    out = torch.full((M, X.shape[1]), float("nan"), device="cuda") if out0 is None else to_dev(out0.copy())
    plan = spmm_kernel.build_plan(rp, len(col))
    spmm_kernel.spmm(rp, c, v, K, Xd, out, plan, accumulate=accumulate)
    torch.cuda.synchronize()
    return out.cpu().numpy()


@pytest.mark.parametrize("F", [1, 3, 4, 8, 16, 17, 32, 47, 64, 100, 128, 172, 233, 256, 384, 512, 520, 1028])
def test_widths_against_oracle(cuda_lib, F):
    rng = np.random.default_rng(F)
    M, K = 1537, 911
    rowptr, col, val = random_csr(rng, M, K, 9, hubs=3, hub_len=900)
    X = rng.standard_normal((K, F)).astype(np.float32)
    out0 = rng.standard_normal((M, F)).astype(np.float32)
    want = oracle.spmm(rowptr, col, val, X, out0.copy())
    got = run_spmm(cuda_lib, rowptr, col, val, K, X, out0, accumulate=True)
    assert_spmm_close(got, want, rowptr, col, val, X, out0)
    want0 = oracle.spmm(rowptr, col, val, X)
    got0 = run_spmm(cuda_lib, rowptr, col, val, K, X, None, accumulate=False)  # output starts as NaN
    assert_spmm_close(got0, want0, rowptr, col, val, X)


def test_bit_exact_when_rows_fit_one_chunk(cuda_lib):
    """F = 128 (one nonzero per warp instruction) and no row longer than a chunk: the kernel
    applies the reference's FMA chain in the reference's order."""
    rng = np.random.default_rng(1)
    M, K, F = 4000, 3000, 128
    rowptr, col, val = random_csr(rng, M, K, 20, hubs=0)
    assert np.diff(rowptr).max() < 400
    X = rng.standard_normal((K, F)).astype(np.float32)
    out0 = rng.standard_normal((M, F)).astype(np.float32)
    want = oracle.spmm(rowptr, col, val, X, out0.copy())
    got = run_spmm(cuda_lib, rowptr, col, val, K, X, out0, accumulate=True)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))
    want0 = oracle.spmm(rowptr, col, val, X)
    got0 = run_spmm(cuda_lib, rowptr, col, val, K, X, None, accumulate=False)
    np.testing.assert_array_equal(got0.view(np.uint32), want0.view(np.uint32))


def test_compiled_reference_fixture(cuda_lib, golden_dir):
    g = np.load(os.path.join(golden_dir, "spmm_ref.npz"))
    got = run_spmm(cuda_lib, g["rowptr"], g["col"], g["val"], g["X"].shape[0], g["X"], g["out0"], accumulate=True)
    np.testing.assert_allclose(got, g["out"], rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("M,K,deg,hubs", [(1, 1, 1, 0), (5, 7, 0, 0), (1, 5000, 0, 1), (3000, 10, 4, 0),
                                          (70000, 300, 1, 0), (257, 100000, 3, 2)])
def test_shapes_edge_cases(cuda_lib, M, K, deg, hubs):
    """Single row, no nonzeros at all, one hub row only, tall-skinny, many empty rows."""
    rng = np.random.default_rng(M * 31 + K)
    rowptr, col, val = random_csr(rng, M, K, deg, hubs=hubs, hub_len=4000, empty_frac=0.5)
    for F in (32, 128):
        X = rng.standard_normal((K, F)).astype(np.float32)
        want = oracle.spmm(rowptr, col, val, X)
        got = run_spmm(cuda_lib, rowptr, col, val, K, X, None, accumulate=False)
        assert_spmm_close(got, want, rowptr, col, val, X)


def test_hub_rows_against_float64(cuda_lib):
    """Rows of 30k nonzeros are cut across ~60 chunks; the error against a float64 product must
    be no worse than the reference order's own."""
    rng = np.random.default_rng(9)
    M, K, F = 64, 40000, 256
    rowptr, col, val = random_csr(rng, M, K, 5, hubs=4, hub_len=30000, empty_frac=0.1)
    X = rng.standard_normal((K, F)).astype(np.float32)
    ref64 = oracle.spmm_f64(rowptr, col, val, X)
    want = oracle.spmm(rowptr, col, val, X)
    got = run_spmm(cuda_lib, rowptr, col, val, K, X, None, accumulate=False)
    assert rel_err(got, ref64) <= 2 * rel_err(want, ref64) + 1e-7
    assert_spmm_close(got, want, rowptr, col, val, X)


def test_strided_operands(cuda_lib):
    """Leading dimensions larger than F (views into wider buffers, as CommBuffer.resize_buffer
    produces) and a misaligned view that must take the scalar path."""
    from gnn_benchmark_b200 import spmm_kernel

    rng = np.random.default_rng(4)
    M, K, F = 700, 500, 64
    rowptr, col, val = random_csr(rng, M, K, 8, hubs=1, hub_len=450)
    Xw = rng.standard_normal((K, F + 8)).astype(np.float32)
    rp, c, v = to_dev(rowptr, torch.int64), to_dev(col, torch.int32), to_dev(val)
    plan = spmm_kernel.build_plan(rp, len(col))
    Xd = to_dev(Xw)
    for off in (0, 8, 3):  # 3: rows start off a 16-byte boundary
        Xv = Xd[:, off:off + F] if off != 3 else Xd[:, 3:3 + F]
        out = torch.zeros(M, F + 4, device="cuda")[:, :F]
        spmm_kernel.spmm(rp, c, v, K, Xv, out, plan, accumulate=False)
        want = oracle.spmm(rowptr, col, val, np.ascontiguousarray(Xv.cpu().numpy()))
        np.testing.assert_allclose(out.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_front_end_forward_backward_like_reference_test(cuda_lib):
    """The reference's own tests/test_spmm.py:70-115: density-0.0007 random 20020 x 1020 matrix,
    128 columns, forward and transposed product, allclose(atol=1e-5) -- here against the oracle
    and a dense float64 product."""
    import scipy.sparse as sp
    from gnn_benchmark_b200 import SparseTensor, SPMM_forward, SPMM_backward

    A = sp.random(20020, 1020, density=0.0007, format="coo", dtype=np.float32, random_state=123)
    rng = np.random.default_rng(0)
    other = rng.random((1020, 128), dtype=np.float32)
    grad_out = rng.standard_normal((20020, 128)).astype(np.float32)
    src = SparseTensor(row=to_dev(A.row, torch.int64), col=to_dev(A.col, torch.int64), value=to_dev(A.data),
                       sparse_sizes=(20020, 1020))
    src.validate()
    out = torch.zeros(20020, 128, device="cuda")
    assert SPMM_forward(src, to_dev(other), out) is None
    SPMM_forward(src, to_dev(other), out)            # accumulates: twice the product
    other_grad = torch.zeros(1020, 128, device="cuda")
    SPMM_backward(src, to_dev(grad_out), other_grad)
    Ad = A.tocsr().astype(np.float64)
    assert torch.allclose(out.cpu(), torch.from_numpy(2 * (Ad @ other)).float(), atol=1e-5)
    assert torch.allclose(other_grad.cpu(), torch.from_numpy(Ad.T @ grad_out).float(), atol=1e-5)
    csr = A.tocsr()
    csr.sort_indices()
    want = oracle.spmm(csr.indptr, csr.indices, csr.data, other)
    np.testing.assert_allclose(out.cpu().numpy(), 2 * want, rtol=RTOL, atol=ATOL)
    csc = A.tocsc()
    csc.sort_indices()
    want_t = oracle.spmm(csc.indptr, csc.indices, csc.data, grad_out)
    np.testing.assert_allclose(other_grad.cpu().numpy(), want_t, rtol=RTOL, atol=ATOL)


@pytest.mark.parametrize("F", [32, 128, 256])
def test_rmat_scale16_forward_and_transposed(cuda_lib, F):
    """Down-scaled instance of the SpMM microbenchmark (R-MAT, symmetrised, GCN-normalised)."""
    from gnn_benchmark_b200 import SparseTensor, SPMM_forward, SPMM_backward, graphgen

    n = 1 << 16
    s, d = graphgen.rmat_edges(16, 16, seed=20261127, device="cuda")
    s, d = graphgen.symmetrize(s, d, n)
    rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
    A = SparseTensor(rowptr=rowptr, col=col, value=val, sparse_sizes=(n, n))
    A.validate()
    g = torch.Generator(device="cuda").manual_seed(F)
    X = torch.randn(n, F, device="cuda", generator=g)
    Y = torch.empty(n, F, device="cuda")
    SPMM_forward(A, X, Y, accumulate=False)
    rp, c, v = rowptr.cpu().numpy(), col.cpu().numpy(), val.cpu().numpy()
    want = oracle.spmm(rp, c, v, X.cpu().numpy())
    np.testing.assert_allclose(Y.cpu().numpy(), want, rtol=RTOL, atol=ATOL)
    ref64 = oracle.spmm_f64(rp, c, v, X.cpu().numpy())
    assert rel_err(Y.cpu().numpy(), ref64) <= 2 * rel_err(want, ref64) + 1e-7
    # transposed: the matrix is symmetric with symmetric values, so A^T G == A G up to rounding order
    Yt = torch.empty(n, F, device="cuda")
    SPMM_backward(A, X, Yt, accumulate=False)
    np.testing.assert_allclose(Yt.cpu().numpy(), want, rtol=RTOL, atol=ATOL)


def test_full_size_properties(cuda_lib):
    """Benchmark-size matrix (R-MAT scale 22, ~1.2e8 nonzeros), checked without a CPU product:
    A @ ones == row sums of the values; linearity A(2x + y) == 2Ax + Ay; accumulate == add."""
    from gnn_benchmark_b200 import SparseTensor, SPMM_forward, graphgen

    n, F = 1 << 22, 32
    s, d = graphgen.rmat_edges(22, 16, seed=20261127, device="cuda")
    s, d = graphgen.symmetrize(s, d, n)
    rowptr, col, val = graphgen.csr_from_edges(s, d, n, n, gcn_normalize=True)
    del s, d
    A = SparseTensor(rowptr=rowptr, col=col, value=val, sparse_sizes=(n, n))
    A.validate()
    ones = torch.ones(n, F, device="cuda")
    Y1 = torch.empty(n, F, device="cuda")
    SPMM_forward(A, ones, Y1, accumulate=False)
    rows = torch.repeat_interleave(torch.arange(n, device="cuda"), rowptr[1:] - rowptr[:-1])
    rowsum = torch.zeros(n, dtype=torch.float64, device="cuda").index_add_(0, rows, val.double())
    del rows
    assert torch.allclose(Y1.double(), rowsum[:, None].expand(n, F), rtol=1e-5, atol=1e-6)
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn(n, F, device="cuda", generator=g)
    y = torch.randn(n, F, device="cuda", generator=g)
    Ax = torch.empty(n, F, device="cuda")
    Ay = torch.empty(n, F, device="cuda")
    Axy = torch.empty(n, F, device="cuda")
    SPMM_forward(A, x, Ax, accumulate=False)
    SPMM_forward(A, y, Ay, accumulate=False)
    SPMM_forward(A, 2 * x + y, Axy, accumulate=False)
    assert torch.allclose(Axy, 2 * Ax + Ay, rtol=1e-4, atol=1e-4)
    acc = Ax.clone()
    SPMM_forward(A, y, acc, accumulate=True)
    assert torch.allclose(acc, Ax + Ay, rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("F", [4, 32, 100, 128, 256, 516])
def test_packed_operand_equals_unpack_then_spmm(cuda_lib, bits, F):
    """gnnagg_spmm_csr_q (codes decoded inside the SpMM) against gnnagg_unpack_dequant_rows followed by
    gnnagg_spmm_csr_f32: bit-identical, accumulate on and off, with empty and ragged peer segments."""
    from gnn_benchmark_b200 import Quantizer_for_all_procs, spmm_kernel

    rng = np.random.default_rng(bits * 1000 + F)
    seg = [0, 37, 37, 401, 402, 1500]
    K, M = seg[-1], 1200
    rowptr, col, val = random_csr(rng, M, K, 7, hubs=2, hub_len=1300)
    halo = rng.standard_normal((K, F)).astype(np.float32)
    q = Quantizer_for_all_procs(len(seg) - 1, bits)
    segd = to_dev(np.asarray(seg, dtype=np.int32))
    epb = 8 // bits
    prow = sum((b - a + epb - 1) // epb for a, b in zip(seg[:-1], seg[1:]))
    codes = torch.zeros(prow, F, dtype=torch.uint8, device="cuda")
    params = torch.zeros(K, 2, device="cuda")
    pb = torch.zeros(K, 2, dtype=torch.bfloat16, device="cuda")
    q.quantize_fp32_to_intX(to_dev(halo), codes, params, segd, params_bf16=pb)
    unpacked = torch.empty(K, F, device="cuda")
    q.dequantize_intX_to_fp32(codes, unpacked, params, segd, params_bf16=pb)
    rp, c, v = to_dev(rowptr, torch.int64), to_dev(col, torch.int32), to_dev(val)
    plan = spmm_kernel.build_plan(rp, len(col))
    base = to_dev(rng.standard_normal((M, F)).astype(np.float32))
    for accumulate in (False, True):
        want, got = base.clone(), base.clone()
        spmm_kernel.spmm(rp, c, v, K, unpacked, want, plan, accumulate=accumulate)
        spmm_kernel.spmm_packed(rp, c, v, K, codes, pb, segd, len(seg) - 1, bits, got, plan, accumulate=accumulate)
        torch.cuda.synchronize()
        np.testing.assert_array_equal(got.cpu().numpy().view(np.uint32), want.cpu().numpy().view(np.uint32))


@pytest.mark.parametrize("M,K,deg,hubs", [(1, 1, 1, 0), (50, 37, 3, 0), (3000, 70000, 5, 2), (20000, 300, 40, 3), (257, 1 << 17, 2, 0)])
def test_csr_to_csc_matches_stable_sort(cuda_lib, M, K, deg, hubs):
    """gnnagg_csr_to_csc against a stable sort by column on the host: column pointers, row order inside a
    column (ascending, duplicates in CSR order) and values, bit for bit."""
    from gnn_benchmark_b200 import SparseTensor

    rng = np.random.default_rng(M + K)
    rowptr, col, val = random_csr(rng, M, K, deg, hubs=hubs, hub_len=min(K, 3000))
    if col.size > 4:  # duplicated entries must keep their order
        col[1] = col[0]
        val[1] = val[0] + 1.0
    A = SparseTensor(rowptr=to_dev(rowptr), col=to_dev(col), value=to_dev(val), sparse_sizes=(M, K))
    colptr, row_T, val_T = A.storage.colptr(), A.storage.row_T(), A.storage.value_T()
    torch.cuda.synchronize()
    rows = np.repeat(np.arange(M), np.diff(rowptr))
    order = np.argsort(col, kind="stable")
    np.testing.assert_array_equal(colptr.cpu().numpy(), np.concatenate([[0], np.cumsum(np.bincount(col, minlength=K))]))
    np.testing.assert_array_equal(row_T.cpu().numpy(), rows[order])
    np.testing.assert_array_equal(val_T.cpu().numpy(), val[order])
