"""K3 parity (bit-exact codes and parameters): quantise+pack / unpack+dequantise kernels through
the C ABI against the CPU oracle and the committed bytes of the reference's compiled module."""
import os

import numpy as np
import pytest
import torch

import oracle
from util import to_dev

pytestmark = pytest.mark.gpu


def bits_eq(a, b):
    """Bit-for-bit equality; a NaN matches any NaN (x86 and the GPU pick different NaN payloads)."""
    a, b = np.ascontiguousarray(a), np.ascontiguousarray(b)
    na, nb = np.isnan(a), np.isnan(b)
    np.testing.assert_array_equal(na, nb)
    np.testing.assert_array_equal(np.where(na, 0, a).view(np.uint32), np.where(nb, 0, b).view(np.uint32))


def gpu_quant_all_procs(x, seg, bits=2, idx=None, want_bf16=True):
    from gnn_benchmark_b200 import Quantizer_for_all_procs

    P = len(seg) - 1
    q = Quantizer_for_all_procs(P, bits)
    segd = to_dev(np.asarray(seg, dtype=np.int32))
    rows = int(seg[-1])
    F = x.shape[1]
    epb = 8 // bits
    prow = int(sum((int(b) - int(a) + epb - 1) // epb for a, b in zip(seg[:-1], seg[1:])))
    codes = torch.full((prow, F), 0xAB, dtype=torch.uint8, device="cuda")
    params = torch.full((rows, 2), float("nan"), device="cuda")
    pb = torch.zeros((rows, 2), dtype=torch.bfloat16, device="cuda") if want_bf16 else None
    q.quantize_fp32_to_intX(to_dev(x), codes, params, segd, params_bf16=pb,
                            gather_idx=None if idx is None else to_dev(idx, torch.int32))
    torch.cuda.synchronize()
    return codes, params, pb, segd, q


SEGS = [[0, 6], [0, 5, 5, 18, 19, 64, 256], [0, 0, 0, 3], [0, 1, 2, 3, 4, 5, 6, 7, 8], [0, 4, 8, 12], [0, 1023]]


@pytest.mark.parametrize("F", [1, 3, 4, 16, 47, 100, 128, 233, 256, 512, 516])
@pytest.mark.parametrize("seg", SEGS)
def test_int2_all_procs_bit_exact(cuda_lib, F, seg):
    rng = np.random.default_rng(F * 7 + len(seg))
    rows = seg[-1]
    x = rng.standard_normal((rows, F)).astype(np.float32)
    x[rows // 2] = 1.5                      # constant row: scale 0 -> 1
    x[0, :] = np.round(x[0] * 2) / 2        # exact ties
    want_codes, want_params = oracle.quantize_int2_for_all_procs(x, seg)
    codes, params, pb, segd, q = gpu_quant_all_procs(x, seg)
    np.testing.assert_array_equal(codes.cpu().numpy(), want_codes)
    bits_eq(params.cpu().numpy(), want_params)
    wire = oracle.bf16_round(want_params)
    bits_eq(pb.float().cpu().numpy(), wire)
    # receive side: parameters come from the bf16 wire buffer
    y = torch.full((rows, F), float("nan"), device="cuda")
    p32 = torch.zeros(rows, 2, device="cuda")
    q.dequantize_intX_to_fp32(codes, y, p32, segd, params_bf16=pb)
    want_y = oracle.dequantize_int2_for_all_procs(want_codes, seg, wire)
    bits_eq(y.cpu().numpy(), want_y)
    bits_eq(p32.cpu().numpy(), wire)
    # and from an fp32 parameter buffer (the reference's call)
    y2 = torch.empty(rows, F, device="cuda")
    q.dequantize_intX_to_fp32(codes, y2, params, segd)
    bits_eq(y2.cpu().numpy(), oracle.dequantize_int2_for_all_procs(want_codes, seg, want_params))


def test_int2_known_answer(cuda_lib):
    X = np.array([[0, 1, 3], [-1, .5, 2], [4, 4, 4], [.25, .75, 1], [10, -10, 0], [1, 2, 2.5]], dtype=np.float32)
    codes, params, pb, _, _ = gpu_quant_all_procs(X, [0, 6])
    assert codes.cpu().tolist() == [[0, 98, 243], [192, 32, 176]]
    assert pb.float().cpu()[:, 1].tolist() == [1, 1, 1, .25, 6.65625, .5]


def test_int2_special_values(cuda_lib):
    """NaN in column 0 sticks, NaN elsewhere is skipped, signed zeros keep the first one met,
    infinities; parameters and codes must still match the oracle bit for bit."""
    F = 128
    rng = np.random.default_rng(2)
    x = rng.standard_normal((12, F)).astype(np.float32)
    x[0, 0] = np.nan
    x[1, 77] = np.nan
    x[2] = np.abs(x[2]); x[2, 5] = 0.0; x[2, 9] = -0.0
    x[3] = np.abs(x[3]); x[3, 5] = -0.0; x[3, 9] = 0.0
    x[4] = -np.abs(x[4]); x[4, 100] = -0.0; x[4, 120] = 0.0
    x[5] = 0.0
    x[6] = -0.0
    x[7, 3] = np.inf
    x[8, 3] = -np.inf
    x[9] = 3e38; x[9, 1] = -3e38           # max - min overflows to inf
    x[10] = 1e-41                           # denormals
    want_codes, want_params = oracle.quantize_int2_for_all_procs(x, [0, 12])
    for xx, FF in ((x, F), (np.ascontiguousarray(x[:, :47]), 47)):
        wc, wp = oracle.quantize_int2_for_all_procs(xx, [0, 12])
        codes, params, _, _, _ = gpu_quant_all_procs(xx, [0, 12])
        bits_eq(params.cpu().numpy(), wp)
        np.testing.assert_array_equal(codes.cpu().numpy(), wc)


def test_fused_gather_pack_equals_gather_then_pack(cuda_lib):
    rng = np.random.default_rng(8)
    n, F = 5000, 256
    x = rng.standard_normal((n, F)).astype(np.float32)
    seg = [0, 700, 700, 1501, 3000]
    idx = rng.integers(0, n, size=3000)
    want_codes, want_params = oracle.quantize_int2_for_all_procs(x[idx], seg)
    codes, params, pb, _, _ = gpu_quant_all_procs(x, seg, idx=idx)
    np.testing.assert_array_equal(codes.cpu().numpy(), want_codes)
    bits_eq(params.cpu().numpy(), want_params)


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_rowpacked_generic_bits_against_compiled_reference_bytes(cuda_lib, golden_dir, bits):
    """x86 generic signature (caller's min / scale): bytes and decoded floats of the compiled
    reference module."""
    from gnn_benchmark_b200 import QuantizerForPureBits

    g = np.load(os.path.join(golden_dir, "quant_rowpacked.npz"))
    x = g["x"]
    rows, F = x.shape
    epb = 8 // bits
    codes = torch.zeros(((rows + epb - 1) // epb, F), dtype=torch.uint8, device="cuda")
    QuantizerForPureBits.quantize_with_given_params(to_dev(x), codes, to_dev(g[f"min{bits}"]),
                                                    to_dev(g[f"scale{bits}"]), bits)
    np.testing.assert_array_equal(codes.cpu().numpy(), g[f"codes{bits}"])
    y = torch.empty(rows, F, device="cuda")
    params = torch.stack((to_dev(g[f"min{bits}"]), to_dev(g[f"scale{bits}"])), 1).contiguous()
    QuantizerForPureBits.dequantize_intX_to_fp32(codes, y, params, bits)
    bits_eq(y.cpu().numpy(), g[f"deq{bits}"])
    # own parameters (ARM-style signature) give the same bytes, since min/scale follow the same rule
    codes2 = torch.zeros_like(codes)
    p2 = torch.zeros(rows, 2, device="cuda")
    QuantizerForPureBits.quantize_fp32_to_intX(to_dev(x), codes2, p2, bits)
    np.testing.assert_array_equal(codes2.cpu().numpy(), g[f"codes{bits}"])


@pytest.mark.parametrize("bits", [4, 8])
@pytest.mark.parametrize("F", [8, 100, 256])
def test_all_procs_int4_int8_against_oracle(cuda_lib, bits, F):
    rng = np.random.default_rng(bits + F)
    seg = [0, 9, 9, 40, 41, 300]
    x = rng.standard_normal((300, F)).astype(np.float32)
    codes, params, pb, segd, q = gpu_quant_all_procs(x, seg, bits=bits)
    epb = 8 // bits
    base = 0
    for a, b in zip(seg[:-1], seg[1:]):
        if b == a:
            continue
        mn = x[a:b].min(1)
        sc = ((x[a:b].max(1) - mn) / np.float32(2 ** bits - 1)).astype(np.float32)
        sc[sc == 0] = 1
        want = oracle.quantize_rowpacked(x[a:b], mn, sc, bits)
        k = (b - a + epb - 1) // epb
        np.testing.assert_array_equal(codes[base:base + k].cpu().numpy(), want)
        bits_eq(params[a:b, 0].cpu().numpy(), mn)
        bits_eq(params[a:b, 1].cpu().numpy(), sc)
        base += k
    assert base == codes.shape[0]


def test_mixed_bits_v1_against_compiled_reference_bytes(cuda_lib, golden_dir):
    from gnn_benchmark_b200 import QuantizerForMixedBits

    g = np.load(os.path.join(golden_dir, "quant_v1.npz"))
    x = g["x"]
    rows, F = x.shape
    bits_t = to_dev(g["bits"])
    rng_t = QuantizerForMixedBits.get_quantized_nodes_feat_range(rows, F, bits_t)
    np.testing.assert_array_equal(rng_t.cpu().numpy(), g["range"])
    params = torch.zeros(rows, 3, device="cuda")
    params[:, 0] = bits_t
    codes = torch.zeros(int(g["range"][-1]), dtype=torch.uint8, device="cuda")
    QuantizerForMixedBits.quantize_fp32_to_intX(to_dev(x), codes, rng_t, params)
    np.testing.assert_array_equal(codes.cpu().numpy(), g["codes"])
    bits_eq(params.cpu().numpy(), g["params"])
    y = torch.empty(rows, F, device="cuda")
    QuantizerForMixedBits.dequantize_intX_to_fp32(codes, y, rng_t, params)
    bits_eq(y.cpu().numpy(), g["deq"])


def test_mixed_bits_reference_unit_test_vector(cuda_lib, golden_dir):
    """tests/test_quantizer.py:57-84 of the reference, literally."""
    import json
    from gnn_benchmark_b200 import QuantizerForMixedBits

    vec = json.load(open(os.path.join(golden_dir, "ref_test_vectors.json")))["quantizer_v1"]
    x = torch.tensor(vec["data"], device="cuda")
    bits_t = torch.tensor(vec["bits"], device="cuda")
    params = torch.empty(5, 3, device="cuda")
    params[:, 0] = bits_t
    rng_t = QuantizerForMixedBits.get_quantized_nodes_feat_range(5, 3, bits_t)
    codes = torch.empty(int(rng_t[-1]), dtype=torch.uint8, device="cuda")
    QuantizerForMixedBits.quantize_fp32_to_intX(x, codes, rng_t, params)
    assert rng_t.cpu().tolist() == vec["range"]
    assert codes.cpu().tolist() == vec["codes"]
    out = torch.empty(5, 3, device="cuda")
    QuantizerForMixedBits.dequantize_intX_to_fp32(codes, out, rng_t, params)
    assert torch.allclose(out, x, atol=0.04)


def test_round_trip_error_bound_large(cuda_lib):
    """2M rows x 256 (halo-exchange size): |dequant(quant(x)) - x| <= scale/2 per row, with the
    sender's fp32 parameters."""
    from gnn_benchmark_b200 import Quantizer_for_all_procs

    rows, F = 1 << 21, 256
    g = torch.Generator(device="cuda").manual_seed(3)
    x = torch.randn(rows, F, device="cuda", generator=g)
    seg = torch.tensor([0, 262143, 262143, 1000001, rows], dtype=torch.int32, device="cuda")
    q = Quantizer_for_all_procs(4, 2)
    prow = sum((b - a + 3) // 4 for a, b in zip(seg.tolist()[:-1], seg.tolist()[1:]))
    codes = torch.empty(prow, F, dtype=torch.uint8, device="cuda")
    params = torch.empty(rows, 2, device="cuda")
    q.quantize_fp32_to_intX(x, codes, params, seg)
    y = torch.empty_like(x)
    q.dequantize_intX_to_fp32(codes, y, params, seg)
    assert torch.equal(params[:, 0], x.min(1).values)
    err = (y - x).abs().max(1).values
    assert bool((err <= params[:, 1] * 0.5 * (1 + 1e-5) + 1e-6).all())


def test_bf16_casts(cuda_lib):
    from gnn_benchmark_b200.communicator import _cast

    g = torch.Generator(device="cuda").manual_seed(0)
    x = torch.randn(100003, device="cuda", generator=g) * 50
    h = torch.empty(100003, dtype=torch.bfloat16, device="cuda")
    _cast(x, h)
    assert torch.equal(h, x.to(torch.bfloat16))
    back = torch.empty_like(x)
    _cast(h, back)
    assert torch.equal(back, h.float())


# ---- SpMM whose epilogue quantises + packs (gnnagg_spmm_quant_pack) ------------------------------------
def _slot_matrix(rng, slots, K, hubs=()):
    """CSR (slots x K): short rows (a post source is one nonzero, a pre destination a few), empty rows,
    optionally rows far longer than an SpMM chunk (hub vertices) at the given positions."""
    deg = rng.integers(0, 7, size=slots)
    deg[rng.random(slots) < 0.3] = 1
    for h, d in hubs:
        deg[h] = min(K, d)
    rowptr = np.concatenate([[0], np.cumsum(deg)]).astype(np.int64)
    col = np.concatenate([np.sort(rng.choice(K, size=d, replace=False)) for d in deg] + [np.zeros(0, np.int64)])
    val = rng.standard_normal(col.shape[0]).astype(np.float32)
    val[rng.random(col.shape[0]) < 0.5] = 1.0  # the plans' matrices are unit-valued
    return rowptr, col.astype(np.int64), val


def _fused(rowptr, col, val, K, X, seg, bits):
    from gnn_benchmark_b200.spmm_kernel import build_plan, spmm_quant_pack

    slots, F, epb = int(seg[-1]), X.shape[1], 8 // bits
    prow = int(sum((int(b) - int(a) + epb - 1) // epb for a, b in zip(seg[:-1], seg[1:])))
    codes = torch.full((prow, F), 0xAB, dtype=torch.uint8, device="cuda")
    params = torch.full((slots, 2), float("nan"), device="cuda")
    pb = torch.zeros((slots, 2), dtype=torch.bfloat16, device="cuda")
    rp = to_dev(rowptr)
    spmm_quant_pack(rp, to_dev(col, torch.int32), to_dev(val), K, to_dev(X), codes, params, pb,
                    to_dev(np.asarray(seg, dtype=np.int32)), len(seg) - 1, bits, build_plan(rp, col.shape[0]))
    torch.cuda.synchronize()
    return codes.cpu().numpy(), params.cpu().numpy(), pb.float().cpu().numpy()


@pytest.mark.parametrize("F", [100, 128, 172, 256, 512])
@pytest.mark.parametrize("seg", [[0, 6], [0, 5, 5, 18, 19, 64, 256], [0, 0, 0, 3], [0, 1023]])
def test_spmm_quant_pack_equals_reference_chain_then_quantise(cuda_lib, F, seg):
    """Codes and parameters of the fused kernel against the oracle's SpMM (sequential FMA chain, the
    reference's order) followed by its int2 quantiser: bit-exact where the kernel keeps that order
    (rows of more than 64 floats that lie inside one chunk)."""
    rng = np.random.default_rng(F + 13 * len(seg))
    slots, K = seg[-1], 700
    rowptr, col, val = _slot_matrix(rng, slots, K)
    X = rng.standard_normal((K, F)).astype(np.float32)
    summed = oracle.spmm(rowptr, col, val, X)
    want_codes, want_params = oracle.quantize_int2_for_all_procs(summed, seg)
    codes, params, pb = _fused(rowptr, col, val, K, X, seg, 2)
    np.testing.assert_array_equal(codes, want_codes)
    bits_eq(params, want_params)
    bits_eq(pb, oracle.bf16_round(want_params))


@pytest.mark.parametrize("bits", [2, 4, 8])
@pytest.mark.parametrize("F", [4, 32, 64, 100, 128, 256, 512])
def test_spmm_quant_pack_equals_two_calls(cuda_lib, bits, F):
    """Same bytes as SPMM_forward into an fp32 buffer followed by gnnagg_quant_pack_rows, for every width,
    with empty rows, ragged peer segments and hub rows cut across several chunks (finished and encoded by
    the fix-up kernel)."""
    from gnn_benchmark_b200 import SparseTensor, SPMM_forward

    rng = np.random.default_rng(bits * 100 + F)
    seg = [0, 37, 37, 201, 333, 640]
    slots, K = seg[-1], 9000
    rowptr, col, val = _slot_matrix(rng, slots, K, hubs=((5, 513), (36, 2000), (37, 1024), (300, 4097), (639, 8999)))
    X = rng.standard_normal((K, F)).astype(np.float32)
    A = SparseTensor(rowptr=to_dev(rowptr), col=to_dev(col), value=to_dev(val), sparse_sizes=(slots, K))
    buf = torch.empty(slots, F, device="cuda")
    SPMM_forward(A, to_dev(X), buf, accumulate=False)
    want_codes, want_params, want_pb, _, _ = gpu_quant_all_procs(buf.cpu().numpy(), seg, bits=bits)
    codes, params, pb = _fused(rowptr, col, val, K, X, seg, bits)
    np.testing.assert_array_equal(codes, want_codes.cpu().numpy())
    bits_eq(params, want_params.cpu().numpy())
    bits_eq(pb, want_pb.float().cpu().numpy())
    # and the hub rows decode to within half a step of the exact sums
    if bits == 2:
        exact = oracle.spmm_f64(rowptr, col, val, X)
        mag = oracle.spmm_f64(rowptr, col, np.abs(val), np.abs(X))
        got = oracle.dequantize_int2_for_all_procs(codes, seg, params)
        for h in (5, 36, 37, 300, 639):
            assert (np.abs(got[h] - exact[h]) <= 0.5 * params[h, 1] * (1 + 1e-5) + 1e-5 * mag[h]).all()


def test_spmm_quant_pack_refuses_unsupported_width(cuda_lib):
    rng = np.random.default_rng(0)
    rowptr, col, val = _slot_matrix(rng, 8, 20)
    with pytest.raises(RuntimeError, match="F %"):
        _fused(rowptr, col, val, 20, rng.standard_normal((20, 6)).astype(np.float32), [0, 8], 2)
