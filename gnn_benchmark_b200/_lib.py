"""ctypes binding of libgnnagg.so, the C-ABI CUDA library (declared in include/gnnagg.h).

The library is the only compute path of this package: if it is missing, or a call returns a
non-zero status, a RuntimeError is raised.  There is no CPU or PyTorch fallback.
"""
import ctypes
import os

import torch

_PKG_DIR = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG_DIR, "libgnnagg.so")

_lib = None

_vp = ctypes.c_void_p
_i64 = ctypes.c_int64
_i32 = ctypes.c_int32
_sz = ctypes.c_size_t

# name -> (restype, argtypes); mirrors include/gnnagg.h one to one
SIGNATURES = {
    "gnnagg_version": (ctypes.c_int, []),
    "gnnagg_error_string": (ctypes.c_char_p, [ctypes.c_int]),
    "gnnagg_spmm_plan_bytes": (_sz, [_i64, _i64]),
    "gnnagg_spmm_plan_build": (ctypes.c_int, [_vp, _i64, _i64, _vp, _sz, _vp]),
    "gnnagg_spmm_scratch_bytes": (_sz, [_i64, _i64, _i32]),
    "gnnagg_spmm_csr_f32": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _i32, _i32, _vp,
                                           _vp, _sz, _vp]),
    "gnnagg_spmm_csr_q": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _i32, _i32, _vp, _i64, _i32, _i32,
                                         _vp, _vp, _sz, _vp]),
    "gnnagg_spmm_csr_f32_static_scratch": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _vp, _i64, _i32,
                                                          _i32, _vp, _vp]),
    "gnnagg_csr_to_csc_workspace_bytes": (_sz, [_i64, _i64, _i64]),
    "gnnagg_csr_to_csc": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _vp, _vp, _vp, _sz, _vp]),
    "gnnagg_csr_validate": (ctypes.c_int, [_vp, _vp, _i64, _i64, _i64, _vp, _vp]),
    "gnnagg_gather_rows_f32": (ctypes.c_int, [_vp, _i64, _vp, _i64, _i32, _vp, _i64, _vp]),
    "gnnagg_push_block": (ctypes.c_int, [_vp, _vp, _sz, _vp]),
    "gnnagg_push_rows": (ctypes.c_int, [_vp, _i64, _vp, _i32, _vp, _i32, _i32, _i32, _vp, _i64, _i64, _vp]),
    "gnnagg_scale_rows_f32": (ctypes.c_int, [_vp, _i64, _vp, _i64, _i32, _i32, _vp, _vp, _i64, _vp]),
    "gnnagg_quant_pack_rows": (ctypes.c_int, [_vp, _i64, _vp, _i32, _vp, _i32, _i64, _i32, _i32, _vp, _vp, _vp, _vp]),
    "gnnagg_spmm_quant_pack_scratch_bytes": (_sz, [_i64, _i64, _i32]),
    "gnnagg_spmm_quant_pack": (ctypes.c_int, [_vp, _vp, _vp, _i64, _i64, _i64, _vp, _i64, _i32, _vp, _i32, _i32, _vp, _vp, _vp,
                                              _vp, _vp, _sz, _vp]),
    "gnnagg_unpack_dequant_rows": (ctypes.c_int, [_vp, _i32, _vp, _i32, _i64, _i32, _vp, _vp, _vp, _i64, _vp]),
    "gnnagg_quant_v1_rows": (ctypes.c_int, [_vp, _i64, _i64, _i32, _vp, _vp, _vp, _vp]),
    "gnnagg_dequant_v1_rows": (ctypes.c_int, [_vp, _i64, _i32, _vp, _vp, _vp, _i64, _vp]),
    "gnnagg_cast_f32_to_bf16": (ctypes.c_int, [_vp, _vp, _i64, _vp]),
    "gnnagg_cast_bf16_to_f32": (ctypes.c_int, [_vp, _vp, _i64, _vp]),
    "gnnagg_dense_workspace_bytes": (_sz, [_i32, _i32]),
    "gnnagg_dense_tf32x3_f32": (ctypes.c_int, [_vp, _i64, _vp, _i64, _vp, _i64, _i64, _i32, _i32, _vp, _i32, _vp, _sz,
                                               _vp]),
    "gnnagg_dense_status": (ctypes.c_int, [_vp, _vp]),
    "gnnagg_dense_status_clear": (ctypes.c_int, [_vp, _vp]),
    "gnnagg_dense_stall_test": (ctypes.c_int, [_i32, _i64]),
    "gnnagg_dense_wgrad_workspace_bytes": (_sz, [_i32, _i32]),
    "gnnagg_dense_wgrad_tf32x3_f32": (ctypes.c_int, [_vp, _i64, _vp, _i64, _i64, _i32, _i32, _vp, _i64, _vp, _sz, _vp]),
    "gnnagg_dropout_ln_relu_partial_bytes": (_sz, [_i32]),
    "gnnagg_dropout_ln_relu_fwd": (ctypes.c_int, [_vp, _i64, _i64, _i32, _vp, _vp, ctypes.c_float, ctypes.c_float,
                                                  ctypes.c_uint64, _vp, _i64, _vp, _vp, _vp]),
    "gnnagg_relu_dropout_fwd": (ctypes.c_int, [_vp, _i64, _i64, _i32, ctypes.c_float, ctypes.c_uint64, _vp, _i64, _vp, _vp]),
    "gnnagg_relu_dropout_bwd": (ctypes.c_int, [_vp, _i64, _vp, _i64, _i32, ctypes.c_float, _vp, _i64, _vp]),
    "gnnagg_dropout_ln_relu_bwd": (ctypes.c_int, [_vp, _i64, _vp, _i64, _vp, _vp, _vp, _vp, _i64, _i32, ctypes.c_float,
                                                  _vp, _i64, _vp, _sz, _vp, _vp, _vp]),
}


def lib():
    """The loaded library.  Raises if libgnnagg.so has not been built
    (`python -m gnn_benchmark_b200.build`)."""
    global _lib
    if _lib is None:
        if not os.path.isfile(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m gnn_benchmark_b200.build` "
                "(nvcc, sm_100a).  This package has no CPU fallback."
            )
        handle = ctypes.CDLL(LIB_PATH)
        for name, (res, args) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc != 0:
        msg = lib().gnnagg_error_string(rc).decode()
        raise RuntimeError(f"libgnnagg {what} failed (status {rc}): {msg}")


def stream_ptr(device=None) -> int:
    """cudaStream_t of torch's current stream on `device`."""
    return torch.cuda.current_stream(device).cuda_stream


def ptr(t) -> int:
    """Device address of a tensor, 0 for None."""
    return 0 if t is None else t.data_ptr()


def require_cuda(*tensors) -> None:
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("libgnnagg kernels take CUDA tensors only (this package has no CPU fallback)")
