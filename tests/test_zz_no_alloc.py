"""The allocation-free SpMM entry point (scratch inside the library) gives what the regular entry
point gives.  For callers that cannot obtain device memory at the call site -- see the comment of
gnnagg_spmm_csr_f32_static_scratch in include/gnnagg.h.  Collected last on purpose: a run that stops
at the first failure has then already run every other test."""
import numpy as np
import pytest
import torch

from util import random_csr, to_dev

pytestmark = pytest.mark.gpu


def _call_static(lib, rp, c, v, K, X, Y, plan, accumulate):
    from gnn_benchmark_b200 import _lib

    M, F = rp.numel() - 1, X.size(1)
    return lib.gnnagg_spmm_csr_f32_static_scratch(rp.data_ptr(), c.data_ptr(), v.data_ptr(), M, K, c.numel(),
                                                  X.data_ptr(), X.stride(0), Y.data_ptr(), Y.stride(0), F,
                                                  1 if accumulate else 0, plan.data_ptr(), _lib.stream_ptr(X.device))


def test_static_scratch_matches_regular_entry_point_twice_in_a_row(cuda_lib):
    from gnn_benchmark_b200 import spmm_kernel

    rng = np.random.default_rng(77)
    M, K = 3000, 9000
    # hub rows longer than a chunk, so partial sums really pass through the scratch buffer
    rowptr, col, val = random_csr(rng, M, K, 12, hubs=5, hub_len=7000)
    rp, c, v = to_dev(rowptr, torch.int64), to_dev(col, torch.int32), to_dev(val)
    plan = spmm_kernel.build_plan(rp, len(col))
    for call, (F, accumulate) in enumerate([(256, False), (128, True)]):  # two calls in a row, one buffer
        X = to_dev(rng.standard_normal((K, F)).astype(np.float32))
        base = to_dev(rng.standard_normal((M, F)).astype(np.float32))
        want = base.clone()
        spmm_kernel.spmm(rp, c, v, K, X, want, plan, accumulate=accumulate)      # caller-provided scratch
        got = base.clone()
        rc = _call_static(cuda_lib, rp, c, v, K, X, got, plan, accumulate)           # built-in scratch
        assert rc == 0, cuda_lib.gnnagg_error_string(rc)
        torch.cuda.synchronize()
        np.testing.assert_allclose(got.cpu().numpy(), want.cpu().numpy(), rtol=1e-5, atol=1e-5,
                                   err_msg=f"call {call}")


def test_static_scratch_rejects_products_beyond_its_capacity(cuda_lib):
    from gnn_benchmark_b200 import spmm_kernel

    rp = torch.zeros(5, dtype=torch.int64, device="cuda")
    plan = spmm_kernel.build_plan(rp, 0)
    x = torch.zeros(4, 256, device="cuda")
    y = torch.zeros(4, 256, device="cuda")
    M, nnz = 1 << 22, 1 << 27  # far more partial-sum slots than 32 MiB holds; nothing is launched
    rc = cuda_lib.gnnagg_spmm_csr_f32_static_scratch(rp.data_ptr(), rp.data_ptr(), x.data_ptr(), M, M, nnz,
                                                     x.data_ptr(), 256, y.data_ptr(), 256, 256, 0, plan.data_ptr(),
                                                     None)
    assert rc == -4
    assert b"built-in buffer" in cuda_lib.gnnagg_error_string(rc)
    torch.cuda.synchronize()
