"""SPMM_forward / SPMM_backward: the reference's SpMM front-end over the CUDA kernel.

Mirrors self_benchmark/a64fx/model/ops/spmm_kernel.py:45-90 of the reference: both calls
ACCUMULATE into the caller's pre-allocated `out` and cache a per-matrix work decomposition on
the SparseTensor (there: greedy per-thread row splits computed by a Python loop, :7-28; here:
the merge-path launch plan built on the GPU by `gnnagg_spmm_plan_build`).
"""
import torch

from . import _lib
from .sparse import SparseTensor

# (device index, stream handle) -> scratch tensor for the partial sums of rows cut across chunks
_scratch = {}


def _get_scratch(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, _lib.stream_ptr(device))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _scratch[key] = buf
    return buf


def build_plan(rowptr: torch.Tensor, nnz: int) -> torch.Tensor:
    """Launch plan (opaque device bytes) for one sparsity pattern; valid for every feature width."""
    _lib.require_cuda(rowptr)
    M = rowptr.numel() - 1
    lib = _lib.lib()
    nbytes = lib.gnnagg_spmm_plan_bytes(M, nnz)
    plan = torch.empty(nbytes, dtype=torch.uint8, device=rowptr.device)
    _lib.check(lib.gnnagg_spmm_plan_build(rowptr.data_ptr(), M, nnz, plan.data_ptr(), nbytes,
                                          _lib.stream_ptr(rowptr.device)), "spmm_plan_build")
    return plan


def spmm(rowptr, col, value, K: int, other: torch.Tensor, out: torch.Tensor, plan: torch.Tensor,
         accumulate: bool = True) -> None:
    """out (+)= CSR(rowptr, col, value)[M,K] @ other[K,F] through the C ABI."""
    _lib.require_cuda(rowptr, col, value, other, out, plan)
    if other.dtype != torch.float32 or out.dtype != torch.float32 or value.dtype != torch.float32:
        # the reference only prints and returns without computing here (spmm.cpp:498-503)
        raise RuntimeError("spmm: sparse values, dense operand and output must be float32")
    if other.dim() != 2 or out.dim() != 2 or other.stride(1) != 1 or out.stride(1) != 1:
        raise RuntimeError("spmm: operands must be 2-D with unit inner stride")
    M = rowptr.numel() - 1
    F = other.size(1)
    if other.size(0) != K or out.size(0) != M or out.size(1) != F:
        raise RuntimeError(f"spmm: shape mismatch A=({M},{K}) other={tuple(other.shape)} out={tuple(out.shape)}")
    if M == 0 or F == 0:
        return
    nnz = col.numel()
    lib = _lib.lib()
    sbytes = lib.gnnagg_spmm_scratch_bytes(M, nnz, F)
    scratch = _get_scratch(out.device, sbytes)
    rc = lib.gnnagg_spmm_csr_f32(rowptr.data_ptr(), _lib.ptr(col), _lib.ptr(value), M, K, nnz, _lib.ptr(other),
                                 other.stride(0) if other.size(0) else F, out.data_ptr(), out.stride(0), F,
                                 1 if accumulate else 0, plan.data_ptr(), scratch.data_ptr(), scratch.numel(),
                                 _lib.stream_ptr(out.device))
    _lib.check(rc, "spmm_csr_f32")


def spmm_packed(rowptr, col, value, K: int, codes: torch.Tensor, params_bf16: torch.Tensor, seg: torch.Tensor,
                num_segments: int, bits: int, out: torch.Tensor, plan: torch.Tensor, accumulate: bool = True) -> None:
    """out (+)= CSR[M,K] @ unpack(codes, params_bf16): the dense operand is the packed halo buffer
    (K wire slots, `seg` = per-peer slot prefix), decoded inside the SpMM."""
    _lib.require_cuda(rowptr, col, value, codes, params_bf16, seg, out, plan)
    if out.dtype != torch.float32 or codes.dtype != torch.uint8 or params_bf16.dtype != torch.bfloat16:
        raise RuntimeError("spmm_packed: expected uint8 codes, bfloat16 params and float32 output")
    M, F = rowptr.numel() - 1, out.size(1)
    if out.size(0) != M or codes.size(-1) != F or out.stride(1) != 1 or not codes.is_contiguous():
        raise RuntimeError("spmm_packed: shape mismatch")
    if M == 0 or F == 0:
        return
    nnz = col.numel()
    lib = _lib.lib()
    sbytes = lib.gnnagg_spmm_scratch_bytes(M, nnz, F)
    scratch = _get_scratch(out.device, sbytes)
    rc = lib.gnnagg_spmm_csr_q(rowptr.data_ptr(), _lib.ptr(col), _lib.ptr(value), M, K, nnz, _lib.ptr(codes),
                               _lib.ptr(params_bf16), seg.data_ptr(), num_segments, bits, out.data_ptr(), out.stride(0),
                               F, 1 if accumulate else 0, plan.data_ptr(), scratch.data_ptr(), scratch.numel(),
                               _lib.stream_ptr(out.device))
    _lib.check(rc, "spmm_csr_q")


def SPMM_forward_packed(src: SparseTensor, codes, params_bf16, seg, num_segments: int, bits: int, out: torch.Tensor,
                        accumulate: bool = True):
    """SPMM_forward whose dense operand is still in its packed wire form (no counterpart call in the
    reference, which always unpacks first)."""
    rowptr, col, value = src.csr()
    plan = src.get_work_range()
    if plan.size(0) == 0:
        plan = build_plan(rowptr, src.nnz())
        src.set_work_range(plan)
    spmm_packed(rowptr, col, value, src.sparse_size(1), codes, params_bf16, seg, num_segments, bits, out, plan, accumulate)
    return None


def SPMM_backward_packed(src: SparseTensor, codes, params_bf16, seg, num_segments: int, bits: int, out: torch.Tensor,
                         accumulate: bool = True):
    """SPMM_backward (src^T @ operand) with a packed dense operand."""
    colptr, row_T, value_T = src.storage.colptr(), src.storage.row_T(), src.storage.value_T()
    plan = src.get_work_range_for_transpose()
    if plan.size(0) == 0:
        plan = build_plan(colptr, src.nnz())
        src.set_work_range_for_transpose(plan)
    spmm_packed(colptr, row_T, value_T, src.sparse_size(0), codes, params_bf16, seg, num_segments, bits, out, plan,
                accumulate)
    return None


def quant_pack_fusable(other: torch.Tensor) -> bool:
    """Can the SpMM-with-packing-epilogue take `other` as its dense operand?  (F a multiple of 4, at most
    512, rows 16-byte aligned; anything else runs SpMM and quantise + pack as two calls.)"""
    F = other.size(1)
    return (other.is_cuda and other.dtype == torch.float32 and other.dim() == 2 and other.stride(1) == 1
            and F % 4 == 0 and 0 < F <= 512 and other.stride(0) % 4 == 0 and other.data_ptr() % 16 == 0)


def spmm_quant_pack(rowptr, col, value, K: int, other: torch.Tensor, codes: torch.Tensor, params: torch.Tensor,
                    params_bf16, seg: torch.Tensor, num_segments: int, bits: int, plan: torch.Tensor) -> None:
    """codes, params = quantise_pack(CSR[M,K] @ other) without the fp32 product ever reaching memory;
    row i of the matrix is wire slot i, `seg` the per-peer slot prefix, `plan` the matrix's SpMM plan."""
    _lib.require_cuda(rowptr, col, value, other, codes, params, params_bf16, seg, plan)
    if other.dtype != torch.float32 or codes.dtype != torch.uint8 or params.dtype != torch.float32:
        raise RuntimeError("spmm_quant_pack: expected float32 operand / params and uint8 codes")
    M, F = rowptr.numel() - 1, other.size(1)
    if other.size(0) != K or params.size(0) != M or codes.size(-1) != F or not codes.is_contiguous() \
            or not params.is_contiguous():
        raise RuntimeError("spmm_quant_pack: shape mismatch")
    if M == 0 or F == 0:
        return
    nnz = col.numel()
    lib = _lib.lib()
    scratch = _get_scratch(other.device, lib.gnnagg_spmm_quant_pack_scratch_bytes(M, nnz, F))
    rc = lib.gnnagg_spmm_quant_pack(rowptr.data_ptr(), _lib.ptr(col), _lib.ptr(value), M, K, nnz, other.data_ptr(),
                                    other.stride(0), F, seg.data_ptr(), num_segments, bits, params.data_ptr(),
                                    _lib.ptr(params_bf16), codes.data_ptr(), plan.data_ptr(), scratch.data_ptr(),
                                    scratch.numel(), _lib.stream_ptr(other.device))
    _lib.check(rc, "spmm_quant_pack")


def SPMM_forward_quant_pack(src: SparseTensor, other, codes, params, params_bf16, seg, num_segments: int, bits: int):
    """quantise_pack(src @ other): SPMM_forward into the send buffer followed by the quantiser
    (model/layers/aggregator.py:48-49 + communicator.py:281-284 of the reference) as one pass."""
    rowptr, col, value = src.csr()
    plan = src.get_work_range()
    if plan.size(0) == 0:
        plan = build_plan(rowptr, src.nnz())
        src.set_work_range(plan)
    spmm_quant_pack(rowptr, col, value, src.sparse_size(1), other, codes, params, params_bf16, seg, num_segments, bits, plan)
    return None


def SPMM_backward_quant_pack(src: SparseTensor, other, codes, params, params_bf16, seg, num_segments: int, bits: int):
    """quantise_pack(src^T @ other) on the cached CSC arrays (the backward twin,
    model/layers/aggregator.py:145-149 + the quantiser)."""
    colptr = src.storage.colptr()
    plan = src.get_work_range_for_transpose()
    if plan.size(0) == 0:
        plan = build_plan(colptr, src.nnz())
        src.set_work_range_for_transpose(plan)
    spmm_quant_pack(colptr, src.storage.row_T(), src.storage.value_T(), src.sparse_size(0), other, codes, params,
                    params_bf16, seg, num_segments, bits, plan)
    return None


def SPMM_forward(src: SparseTensor, other: torch.Tensor, out: torch.Tensor, accumulate: bool = True):
    """out += src @ other.  Returns None, like the reference (spmm_kernel.py:45-67).

    `accumulate=False` (an extension) writes out = src @ other without reading `out`."""
    rowptr, col, value = src.csr()
    plan = src.get_work_range()
    if plan.size(0) == 0:
        plan = build_plan(rowptr, src.nnz())
        src.set_work_range(plan)
    spmm(rowptr, col, value, src.sparse_size(1), other, out, plan, accumulate)
    return None


def SPMM_backward(src: SparseTensor, other: torch.Tensor, out: torch.Tensor, accumulate: bool = True):
    """out += src^T @ other via the cached CSC arrays (spmm_kernel.py:71-90)."""
    colptr = src.storage.colptr()
    row_T = src.storage.row_T()
    value_T = src.storage.value_T()
    plan = src.get_work_range_for_transpose()
    if plan.size(0) == 0:
        plan = build_plan(colptr, src.nnz())
        src.set_work_range_for_transpose(plan)
    spmm(colptr, row_T, value_T, src.sparse_size(0), other, out, plan, accumulate)
    return None
