"""The C-ABI library loads without a GPU and exports exactly what include/gnnagg.h declares."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "gnnagg.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(gnnagg_[a-z0-9_]+)\s*\(", text)))


def test_every_declared_symbol_is_exported_and_bound(cuda_lib):
    from gnn_benchmark_b200 import _lib

    names = declared_symbols()
    assert len(names) >= 14
    for n in names:
        assert hasattr(cuda_lib, n), f"{n} declared in gnnagg.h but not exported"
    assert sorted(_lib.SIGNATURES) == names, "ctypes signature table and header disagree"


def test_host_only_entry_points(cuda_lib):
    assert cuda_lib.gnnagg_version() >= 100
    assert cuda_lib.gnnagg_error_string(0) == b"ok"
    assert cuda_lib.gnnagg_spmm_plan_bytes(1000, 16000) % 256 == 0
    assert cuda_lib.gnnagg_spmm_plan_bytes(-1, 5) == 0
    small = cuda_lib.gnnagg_spmm_scratch_bytes(1000, 16000, 32)
    big = cuda_lib.gnnagg_spmm_scratch_bytes(1000, 16000, 256)
    assert 0 < small < big
    # widths beyond one column strip reuse the strip-sized scratch
    assert cuda_lib.gnnagg_spmm_scratch_bytes(1000, 16000, 4096) == cuda_lib.gnnagg_spmm_scratch_bytes(1000, 16000, 512)


def test_argument_errors_are_status_codes_not_crashes(cuda_lib):
    rc = cuda_lib.gnnagg_spmm_csr_f32(None, None, None, 4, 4, 1, None, 4, None, 4, 4, 0, None, None, 0, None)
    assert rc == -1 and b"null" in cuda_lib.gnnagg_error_string(rc)
    rc = cuda_lib.gnnagg_spmm_csr_f32(None, None, None, -1, 4, 1, None, 4, None, 4, 4, 0, None, None, 0, None)
    assert rc == -1
    assert cuda_lib.gnnagg_quant_pack_rows(None, 4, None, 4, None, 1, 8, 2, 0, None, None, None, None) == -1
    seg = (ctypes.c_int32 * 2)(0, 8)
    rc = cuda_lib.gnnagg_quant_pack_rows(None, 4, None, 4, ctypes.addressof(seg), 1, 8, 3, 0, None, None, None, None)
    assert rc == -1 and b"bits" in cuda_lib.gnnagg_error_string(rc)
    rc = cuda_lib.gnnagg_unpack_dequant_rows(None, 4, ctypes.addressof(seg), 5000, 8, 2, None, None, None, 4, None)
    assert rc == -2
    # zero-sized work is a no-op that never touches the device
    assert cuda_lib.gnnagg_gather_rows_f32(None, 0, None, 0, 16, None, 0, None) == 0
    assert cuda_lib.gnnagg_spmm_csr_f32(None, None, None, 0, 0, 0, None, 0, None, 0, 16, 0, None, None, 0, None) == 0


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    from gnn_benchmark_b200 import _lib

    monkeypatch.setattr(_lib, "_lib", None)
    monkeypatch.setattr(_lib, "LIB_PATH", str(tmp_path / "nope.so"))
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        _lib.lib()


def test_cpu_tensors_are_refused():
    import torch
    from gnn_benchmark_b200 import SparseTensor, SPMM_forward

    a = SparseTensor(row=torch.tensor([0, 1]), col=torch.tensor([1, 0]), sparse_sizes=(2, 2))
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        SPMM_forward(a, torch.ones(2, 4), torch.zeros(2, 4))


def test_dense_side_wrappers_refuse_cpu_tensors():
    """The dense-side front-ends have no CPU path either."""
    import pytest
    import torch

    from gnn_benchmark_b200 import dense, norm

    x, w = torch.randn(8, 16), torch.randn(4, 16)
    for call in (lambda: dense.linear(x, w), lambda: dense.wgrad(torch.randn(8, 4), x),
                 lambda: dense.scale_rows(x, torch.ones(8)),
                 lambda: norm.dropout_ln_relu(x, torch.ones(16), torch.zeros(16), 0.0, False),
                 lambda: norm.relu_dropout_(x, 0.0, False)):
        with pytest.raises(RuntimeError):
            call()
