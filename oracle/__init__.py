"""TEST INFRASTRUCTURE: numpy front-end of the CPU oracle (`oracle/gnnagg_oracle.c`).

Only `tests/`, `__graft_entry__.smoke()` and the `cpu_baseline` / `--impl reference`
legs of `bench.py` may import this package.  The product package
(`gnn_benchmark_b200`) never does: it fails loudly when its CUDA library is missing.

Every function takes and returns numpy arrays; the arithmetic lives in the C file,
whose comments cite the reference lines each function restates.
"""
import ctypes
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "liboracle.so")
_lib = None

_i64p = ctypes.POINTER(ctypes.c_int64)
_i32p = ctypes.POINTER(ctypes.c_int32)
_f32p = ctypes.POINTER(ctypes.c_float)
_f64p = ctypes.POINTER(ctypes.c_double)
_u8p = ctypes.POINTER(ctypes.c_uint8)


def build(force: bool = False) -> str:
    """Compile liboracle.so with gcc (seconds)."""
    src = os.path.join(_HERE, "gnnagg_oracle.c")
    if force or not os.path.isfile(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B", "liboracle.so"], check=True, stdout=subprocess.DEVNULL)
    return _LIB_PATH


def lib():
    global _lib
    if _lib is None:
        build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.oracle_num_threads.restype = ctypes.c_int
    return _lib


def _p(a, t):
    return a.ctypes.data_as(t)


def _c(a, dt):
    return np.ascontiguousarray(a, dtype=dt)


def num_threads() -> int:
    return int(lib().oracle_num_threads())


def spmm(rowptr, col, val, X, out=None):
    """out (+)= A @ X in the reference's order; returns out (fp32, accumulated in place)."""
    rowptr, col, val, X = _c(rowptr, np.int64), _c(col, np.int64), _c(val, np.float32), _c(X, np.float32)
    M, F = rowptr.shape[0] - 1, X.shape[1]
    if out is None:
        out = np.zeros((M, F), dtype=np.float32)
    assert out.dtype == np.float32 and out.flags.c_contiguous and out.shape == (M, F)
    lib().oracle_spmm_csr_f32(_p(rowptr, _i64p), _p(col, _i64p), _p(val, _f32p), ctypes.c_int64(M),
                              _p(X, _f32p), _p(out, _f32p), ctypes.c_int64(F))
    return out


def spmm_f64(rowptr, col, val, X):
    rowptr, col, val, X = _c(rowptr, np.int64), _c(col, np.int64), _c(val, np.float32), _c(X, np.float32)
    M, F = rowptr.shape[0] - 1, X.shape[1]
    out = np.zeros((M, F), dtype=np.float64)
    lib().oracle_spmm_csr_f64acc(_p(rowptr, _i64p), _p(col, _i64p), _p(val, _f32p), ctypes.c_int64(M),
                                 _p(X, _f32p), _p(out, _f64p), ctypes.c_int64(F))
    return out


def distribute_work_for_row(rowptr, val, num_threads_on_row):
    rowptr, val = _c(rowptr, np.int64), _c(val, np.float32)
    M = rowptr.shape[0] - 1
    splits = np.empty(num_threads_on_row + 1, dtype=np.int32)
    lib().oracle_distribute_work_for_row(_p(rowptr, _i64p), _p(val, _f32p), ctypes.c_int64(M),
                                         ctypes.c_int32(num_threads_on_row), _p(splits, _i32p))
    return splits


def packed_rows(seg, per_byte=4):
    seg = np.asarray(seg, dtype=np.int64)
    n = np.diff(seg)
    return int(((n + per_byte - 1) // per_byte).sum())


def quantize_int2_for_all_procs(x, seg):
    """-> (codes uint8 (sum ceil(n_p/4), F), params fp32 (rows, 2) [zero_point, scale])."""
    x, seg = _c(x, np.float32), _c(seg, np.int32)
    rows, F = x.shape
    assert seg[-1] == rows
    codes = np.zeros((packed_rows(seg), F), dtype=np.uint8)
    params = np.zeros((rows, 2), dtype=np.float32)
    lib().oracle_quantize_int2_for_all_procs(_p(x, _f32p), ctypes.c_int64(F), _p(seg, _i32p),
                                             ctypes.c_int32(len(seg) - 1), _p(codes, _u8p), _p(params, _f32p))
    return codes, params


def dequantize_int2_for_all_procs(codes, seg, params):
    codes, seg, params = _c(codes, np.uint8), _c(seg, np.int32), _c(params, np.float32)
    rows, F = int(seg[-1]), codes.shape[1]
    y = np.zeros((rows, F), dtype=np.float32)
    lib().oracle_dequantize_int2_for_all_procs(_p(codes, _u8p), ctypes.c_int64(F), _p(seg, _i32p),
                                               ctypes.c_int32(len(seg) - 1), _p(params, _f32p), _p(y, _f32p))
    return y


def quantize_rowpacked(x, mn, scale, bits):
    x, mn, scale = _c(x, np.float32), _c(mn, np.float32), _c(scale, np.float32)
    rows, F = x.shape
    epb = 8 // bits
    codes = np.zeros(((rows + epb - 1) // epb, F), dtype=np.uint8)
    lib().oracle_quantize_rowpacked(_p(x, _f32p), ctypes.c_int64(rows), ctypes.c_int64(F), _p(mn, _f32p),
                                    _p(scale, _f32p), ctypes.c_int32(bits), _p(codes, _u8p))
    return codes


def dequantize_rowpacked(codes, rows, mn, scale, bits, fused=True):
    codes, mn, scale = _c(codes, np.uint8), _c(mn, np.float32), _c(scale, np.float32)
    F = codes.shape[1]
    y = np.zeros((rows, F), dtype=np.float32)
    lib().oracle_dequantize_rowpacked(_p(codes, _u8p), ctypes.c_int64(rows), ctypes.c_int64(F), _p(mn, _f32p),
                                      _p(scale, _f32p), ctypes.c_int32(bits), _p(y, _f32p), ctypes.c_int32(1 if fused else 0))
    return y


def quantized_nodes_feat_range(bits_per_row, F):
    """[0, cumsum(ceil(bits*F/8))] int64 -- quantizer.py:69-76 of the reference."""
    b = np.asarray(bits_per_row, dtype=np.int64)
    ln = (b * F + 7) // 8
    return np.concatenate([[0], np.cumsum(ln)]).astype(np.int64)


def quantize_v1(x, bits_per_row):
    """-> (codes uint8 (range[-1],), params fp32 (rows,3) [bits, zp, scale], range int64)."""
    x = _c(x, np.float32)
    rows, F = x.shape
    rng = quantized_nodes_feat_range(bits_per_row, F)
    params = np.zeros((rows, 3), dtype=np.float32)
    params[:, 0] = np.asarray(bits_per_row, dtype=np.float32)
    codes = np.zeros(int(rng[-1]), dtype=np.uint8)
    lib().oracle_quantize_v1(_p(x, _f32p), ctypes.c_int64(rows), ctypes.c_int64(F), _p(rng, _i64p),
                             _p(params, _f32p), _p(codes, _u8p))
    return codes, params, rng


def dequantize_v1(codes, rows, F, rng, params, fused=True):
    codes, rng, params = _c(codes, np.uint8), _c(rng, np.int64), _c(params, np.float32)
    y = np.zeros((rows, F), dtype=np.float32)
    lib().oracle_dequantize_v1(_p(codes, _u8p), ctypes.c_int64(rows), ctypes.c_int64(F), _p(rng, _i64p),
                               _p(params, _f32p), _p(y, _f32p), ctypes.c_int32(1 if fused else 0))
    return y


def bf16_round(x):
    x = _c(x, np.float32)
    y = np.empty_like(x)
    lib().oracle_bf16_round(_p(x.reshape(-1), _f32p), ctypes.c_int64(x.size), _p(y.reshape(-1), _f32p))
    return y


def load_reference_module():
    """Import the reference's compiled `computation_ops` from oracle/_ref, or None.

    None when it was never built (no reference checkout at build time) or the host CPU
    lacks the AVX-512 subsets it was compiled for."""
    import importlib.util

    path = os.path.join(_HERE, "_ref", "computation_ops.so")
    if not os.path.isfile(path):
        return None
    from .build_ref import cpu_has_avx512

    if not cpu_has_avx512():
        return None
    import torch  # noqa: F401  (the module links against libtorch)

    spec = importlib.util.spec_from_file_location("computation_ops", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod
