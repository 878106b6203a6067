"""Pins the CPU oracle (oracle/gnnagg_oracle.c) to the reference: committed golden outputs of the
reference's compiled x86 module, the literal vectors of the reference's unit tests, and -- when
oracle/_ref is present -- the compiled module itself."""
import json
import os

import numpy as np
import pytest
import torch

import oracle


def test_v1_golden_bytes_of_reference_unit_test(golden_dir):
    vec = json.load(open(os.path.join(golden_dir, "ref_test_vectors.json")))["quantizer_v1"]
    x = np.array(vec["data"], dtype=np.float32)
    codes, params, rng = oracle.quantize_v1(x, vec["bits"])
    assert codes.tolist() == vec["codes"]
    assert rng.tolist() == vec["range"]
    mn = x.min(1)
    np.testing.assert_array_equal(params[:, 1], mn)
    np.testing.assert_allclose(params[:, 2], (x.max(1) - mn) / (2.0 ** np.array(vec["bits"]) - 1), rtol=1e-6)
    y = oracle.dequantize_v1(codes, 5, 3, rng, params)
    np.testing.assert_allclose(y, x, atol=0.04)  # what tests/test_quantizer.py:87-114 expects (allclose)


def test_feat_range_vectors(golden_dir):
    for n, F, bits, expect in json.load(open(os.path.join(golden_dir, "ref_test_vectors.json")))["feat_range"]["cases"]:
        assert oracle.quantized_nodes_feat_range(bits, F).tolist() == expect


def test_v1_against_compiled_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "quant_v1.npz"))
    codes, params, rng = oracle.quantize_v1(g["x"], g["bits"].astype(np.int64))
    np.testing.assert_array_equal(rng, g["range"])
    np.testing.assert_array_equal(codes, g["codes"])
    np.testing.assert_array_equal(params.view(np.uint32), g["params"].view(np.uint32))
    y = oracle.dequantize_v1(codes, g["x"].shape[0], g["x"].shape[1], rng, params, fused=True)
    np.testing.assert_array_equal(y.view(np.uint32), g["deq"].view(np.uint32))


@pytest.mark.parametrize("bits", [2, 4, 8])
def test_rowpacked_against_compiled_reference_fixture(golden_dir, bits):
    g = np.load(os.path.join(golden_dir, "quant_rowpacked.npz"))
    x = g["x"]
    codes = oracle.quantize_rowpacked(x, g[f"min{bits}"], g[f"scale{bits}"], bits)
    np.testing.assert_array_equal(codes, g[f"codes{bits}"])
    y = oracle.dequantize_rowpacked(codes, x.shape[0], g[f"min{bits}"], g[f"scale{bits}"], bits, fused=True)
    np.testing.assert_array_equal(y.view(np.uint32), g[f"deq{bits}"].view(np.uint32))


def test_spmm_against_compiled_reference_fixture(golden_dir):
    g = np.load(os.path.join(golden_dir, "spmm_ref.npz"))
    out = oracle.spmm(g["rowptr"], g["col"], g["val"], g["X"], g["out0"].copy())
    np.testing.assert_array_equal(out.view(np.uint32), g["out"].view(np.uint32))
    # and it is a sane product: within fp32 noise of the float64 result
    ref64 = oracle.spmm_f64(g["rowptr"], g["col"], g["val"], g["X"]) + g["out0"]
    np.testing.assert_allclose(out, ref64, rtol=1e-5, atol=1e-5)


def test_int2_known_answer():
    """Hand-checkable case: ties-to-even (1.5 -> 2), constant row (scale 0 -> 1), 6 rows = one
    full group and a tail group of two."""
    X = np.array([[0, 1, 3], [-1, .5, 2], [4, 4, 4], [.25, .75, 1], [10, -10, 0], [1, 2, 2.5]], dtype=np.float32)
    codes, params = oracle.quantize_int2_for_all_procs(X, [0, 6])
    assert codes.tolist() == [[0, 98, 243], [192, 32, 176]]
    np.testing.assert_array_equal(params[:, 0], [0, -1, 4, .25, -10, 1])
    np.testing.assert_array_equal(params[:, 1], np.array([1, 1, 1, .25, 20 / 3, .5], dtype=np.float32))
    wire = oracle.bf16_round(params)
    assert wire[4, 1] == 6.65625 and np.array_equal(np.delete(wire, 4, 0), np.delete(params, 4, 0))


def test_int2_segments_equal_concatenated_single_segments():
    """for_all_procs(x, ranges) == concat_p quantize(x[range_p]): the invariant the reference's
    tests/test_quantization_ops.py:223-245 prints; single segments use the generic row-packed
    routine that is pinned to the compiled x86 module above."""
    rng = np.random.default_rng(3)
    x = rng.standard_normal((256, 233)).astype(np.float32)
    seg = np.array([0, 5, 5, 18, 19, 64, 256], dtype=np.int32)
    codes, params = oracle.quantize_int2_for_all_procs(x, seg)
    base = 0
    for a, b in zip(seg[:-1], seg[1:]):
        n = int(b - a)
        if n == 0:
            continue
        c = oracle.quantize_rowpacked(x[a:b], params[a:b, 0], params[a:b, 1], 2)
        np.testing.assert_array_equal(c, codes[base: base + (n + 3) // 4])
        base += (n + 3) // 4
    assert base == codes.shape[0]
    y = oracle.dequantize_int2_for_all_procs(codes, seg, params)
    assert np.all(np.abs(y - x) <= params[:, 1:2] * 0.5 * (1 + 1e-5) + 1e-6)


def test_int2_edge_cases():
    x = np.array([[np.nan, 1, 2, 3], [1, np.nan, 3, 2], [0.0, -0.0, 0.0, 0.0], [-0.0, 0.0, 5, 1]], dtype=np.float32)
    codes, params = oracle.quantize_int2_for_all_procs(x, [0, 4])
    assert np.isnan(params[0]).all()                 # NaN in column 0 sticks
    assert params[1, 0] == 1 and params[1, 1] == np.float32(2) / np.float32(3)  # NaN elsewhere is skipped
    assert params[2, 1] == 1.0                       # all zeros: scale 0 -> 1
    assert np.signbit(params[3, 0]) and not np.signbit(params[2, 0])  # first zero met is kept
    # empty input / empty segments
    c, p = oracle.quantize_int2_for_all_procs(np.zeros((0, 8), np.float32), [0, 0, 0])
    assert c.shape == (0, 8) and p.shape == (0, 2)


def test_bf16_round_matches_torch():
    rng = np.random.default_rng(5)
    x = np.concatenate([rng.standard_normal(4096).astype(np.float32) * 100,
                        np.array([0, -0.0, np.inf, -np.inf, 1e-40, 3.3895314e38], dtype=np.float32)])
    ours = oracle.bf16_round(x)
    theirs = torch.from_numpy(x).to(torch.bfloat16).to(torch.float32).numpy()
    np.testing.assert_array_equal(ours.view(np.uint32), theirs.view(np.uint32))


def test_distribute_work_for_row():
    # 4 rows with 3, 1, 1, 3 unit values, 2 threads: target = 4, the cut is placed before the row
    # that makes the running sum exceed it (spmm_kernel.py:18-25)
    rowptr = np.array([0, 3, 4, 5, 8], dtype=np.int64)
    s = oracle.distribute_work_for_row(rowptr, np.ones(8, np.float32), 2)
    assert s.tolist() == [0, 2, 4]


def test_compiled_reference_module_if_present():
    ref = oracle.load_reference_module()
    if ref is None:
        pytest.skip("oracle/_ref not built on this machine")
    rng = np.random.default_rng(11)
    import scipy.sparse as sp
    A = sp.random(500, 300, density=0.02, format="csr", dtype=np.float32, random_state=2)
    A.sort_indices()
    X = rng.standard_normal((300, 100)).astype(np.float32)
    out = torch.zeros(500, 100)
    splits = oracle.distribute_work_for_row(A.indptr, np.ones_like(A.data), torch.get_num_threads())
    ref.spmm(torch.from_numpy(A.indptr.astype(np.int64)), torch.from_numpy(A.indices.astype(np.int64)),
             torch.from_numpy(A.data), torch.from_numpy(X), out, 500, torch.from_numpy(splits),
             torch.tensor([0, 100], dtype=torch.int32))
    np.testing.assert_array_equal(oracle.spmm(A.indptr, A.indices, A.data, X), out.numpy())
