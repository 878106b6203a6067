"""Quantizer front-ends with the reference's class and method names over the CUDA codec.

Mirrors self_benchmark/a64fx/quantizer.py:10-95.  All tensors are CUDA tensors; outputs are
pre-allocated by the caller and written in place, as in the reference.
"""
import math

import torch
from torch import Tensor

from . import _lib


def _one_segment(rows: int, device) -> Tensor:
    return torch.tensor([0, rows], dtype=torch.int32, device=device)


def _quant_pack(data_fp32, data_intX, params, seg, P, bits, params_given=False, params_bf16=None, gather_idx=None,
                rows=None):
    _lib.require_cuda(data_fp32, data_intX, params, seg, params_bf16, gather_idx)
    if data_fp32.dtype != torch.float32 or data_intX.dtype != torch.uint8 or params.dtype != torch.float32:
        raise RuntimeError("quantize: expected float32 input / params and uint8 output")
    if seg.dtype != torch.int32:
        raise RuntimeError("quantize: work_range_per_proc must be int32")
    if data_fp32.stride(-1) != 1 or not data_intX.is_contiguous() or not params.is_contiguous():
        raise RuntimeError("quantize: input rows must be dense, codes and params contiguous")
    F = data_fp32.size(1)
    rows = (data_fp32.size(0) if gather_idx is None else gather_idx.numel()) if rows is None else rows
    rc = _lib.lib().gnnagg_quant_pack_rows(
        _lib.ptr(data_fp32), data_fp32.stride(0) if data_fp32.size(0) > 1 else max(F, data_fp32.stride(0)),
        _lib.ptr(gather_idx), F, seg.data_ptr(), P, rows, bits, 1 if params_given else 0, _lib.ptr(params),
        _lib.ptr(params_bf16), _lib.ptr(data_intX), _lib.stream_ptr(data_fp32.device))
    _lib.check(rc, "quant_pack_rows")


def _unpack_dequant(data_intX, data_fp32, params, seg, P, bits, params_bf16=None):
    _lib.require_cuda(data_intX, data_fp32, params, seg, params_bf16)
    if data_fp32.dtype != torch.float32 or data_intX.dtype != torch.uint8:
        raise RuntimeError("dequantize: expected uint8 input and float32 output")
    if data_fp32.stride(-1) != 1 or not data_intX.is_contiguous():
        raise RuntimeError("dequantize: output rows must be dense and codes contiguous")
    F = data_fp32.size(1)
    rows = data_fp32.size(0)
    rc = _lib.lib().gnnagg_unpack_dequant_rows(
        _lib.ptr(data_intX), F, seg.data_ptr(), P, rows, bits, _lib.ptr(params), _lib.ptr(params_bf16),
        _lib.ptr(data_fp32), data_fp32.stride(0) if rows > 1 else max(F, data_fp32.stride(0)),
        _lib.stream_ptr(data_fp32.device))
    _lib.check(rc, "unpack_dequant_rows")


class QuantizerForPureBits(object):
    """One segment, row-packed, 8/num_bits rows per byte (quantizer.py:10-47).

    `quant_params` is (rows, 2) fp32 [zero_point, scale], computed by the kernel (the ARM
    signature quantizer.py:18 calls).  The ARM kernel ignores `num_bits` and always packs 2 bits
    (quantization_arm.cpp:314-315); here num_bits in {2, 4, 8} is honoured, with the x86 generic
    kernel's layout (quantization_x86.cpp:17-102)."""

    def __init__(self):
        pass

    @staticmethod
    def quantize_fp32_to_intX(data_fp32, data_intX, quant_params, num_bits=8):
        seg = _one_segment(data_fp32.size(0), data_fp32.device)
        _quant_pack(data_fp32, data_intX.view(-1, data_fp32.size(1)), quant_params, seg, 1, num_bits)

    @staticmethod
    def quantize_with_given_params(data_fp32, data_intX, min_, scale, num_bits=8):
        """x86 generic signature: caller supplies per-row min and scale (quantization_x86.h:5)."""
        params = torch.stack((min_.to(torch.float32), scale.to(torch.float32)), dim=1).contiguous()
        seg = _one_segment(data_fp32.size(0), data_fp32.device)
        _quant_pack(data_fp32, data_intX.view(-1, data_fp32.size(1)), params, seg, 1, num_bits, params_given=True)

    @staticmethod
    def dequantize_intX_to_fp32(data_intX, data_fp32, dequant_params, num_bits=8):
        seg = _one_segment(data_fp32.size(0), data_fp32.device)
        _unpack_dequant(data_intX.view(-1, data_fp32.size(1)), data_fp32, dequant_params.contiguous(), seg, 1, num_bits)

    @staticmethod
    def get_quantized_buffer_size(num_comm_nodes, num_bits, feat_len):
        return math.ceil(num_comm_nodes / float(8 / num_bits)) * feat_len


class QuantizerForMixedBits(object):
    """Per-row bit widths 8/4/2, column-packed inside a row (quantizer.py:50-76)."""

    @staticmethod
    def quantize_fp32_to_intX(data_fp32, data_int8, quantized_nodes_feat_range, quantized_params):
        _lib.require_cuda(data_fp32, data_int8, quantized_nodes_feat_range, quantized_params)
        if quantized_nodes_feat_range.dtype != torch.int64 or not quantized_params.is_contiguous():
            raise RuntimeError("quantize_v1: range must be int64 and params contiguous (rows, 3) float32")
        rows, F = data_fp32.shape
        rc = _lib.lib().gnnagg_quant_v1_rows(_lib.ptr(data_fp32), data_fp32.stride(0) if rows > 1 else F, rows, F,
                                             quantized_nodes_feat_range.data_ptr(), quantized_params.data_ptr(),
                                             _lib.ptr(data_int8), _lib.stream_ptr(data_fp32.device))
        _lib.check(rc, "quant_v1_rows")

    @staticmethod
    def dequantize_intX_to_fp32(data_int8, data_fp32, quantized_nodes_feat_range, dequantized_params):
        _lib.require_cuda(data_fp32, data_int8, quantized_nodes_feat_range, dequantized_params)
        rows, F = data_fp32.shape
        rc = _lib.lib().gnnagg_dequant_v1_rows(_lib.ptr(data_int8), rows, F, quantized_nodes_feat_range.data_ptr(),
                                               dequantized_params.contiguous().data_ptr(), _lib.ptr(data_fp32),
                                               data_fp32.stride(0) if rows > 1 else F,
                                               _lib.stream_ptr(data_fp32.device))
        _lib.check(rc, "dequant_v1_rows")

    @staticmethod
    def get_quantized_nodes_feat_range(num_nodes: int, feat_len: int, nodes_num_bits_tensor: Tensor):
        # bytes per row = ceil(bits * feat_len / 8); range = [0, cumsum] (quantizer.py:69-76)
        quantized_nodes_feat_len = torch.ceil(nodes_num_bits_tensor * feat_len / 8.0)
        quantized_nodes_feat_range = torch.empty((num_nodes + 1), dtype=torch.int64,
                                                 device=nodes_num_bits_tensor.device)
        quantized_nodes_feat_range[0] = 0
        torch.cumsum(quantized_nodes_feat_len, dim=0, out=quantized_nodes_feat_range[1:])
        return quantized_nodes_feat_range


class Quantizer_for_all_procs(object):
    """The live halo codec: all peer segments in one call (quantizer.py:78-95).

    The reference's kernel packs 2 bits whatever `num_bits` says (quantization_arm.cpp:380-381);
    here num_bits in {2, 4, 8} selects the packing, 2 being the reference's behaviour."""

    ctx = None

    def __init__(self, world_size, num_bits) -> None:
        self.num_bits = num_bits
        self.world_size = world_size
        Quantizer_for_all_procs.ctx = self

    def _bits(self):
        return self.num_bits if self.num_bits in (2, 4, 8) else 2

    def quantize_fp32_to_intX(self, data_fp32, data_int8, quantized_params, quantized_work_range_per_proc,
                              params_bf16=None, gather_idx=None):
        """`params_bf16` (optional, (rows,2) bf16) also receives the wire copy of the parameters;
        `gather_idx` (optional int32) quantises data_fp32[gather_idx] without materialising it."""
        _quant_pack(data_fp32, data_int8, quantized_params, quantized_work_range_per_proc, self.world_size,
                    self._bits(), params_bf16=params_bf16, gather_idx=gather_idx)

    def dequantize_intX_to_fp32(self, data_int8, data_fp32, quantized_params, dequantized_work_range_per_proc,
                                params_bf16=None):
        """`params_bf16` (optional): read the parameters from the bf16 wire buffer and store their
        fp32 widening into quantized_params."""
        _unpack_dequant(data_int8, data_fp32, quantized_params, dequantized_work_range_per_proc, self.world_size,
                        self._bits(), params_bf16=params_bf16)

    def get_quantized_splits(self, num_comm_nodes):
        return math.ceil(num_comm_nodes / float(8 / self._bits()))
