"""ctypes binding of libfpq_b200.so (the C ABI declared in include/fpq_b200.h).

There is no CPU implementation behind these calls: if the shared library is missing
or a tensor is not on a CUDA device, the call raises.
"""
from __future__ import annotations

import ctypes
import os
from ctypes import c_int, c_int32, c_int64, c_void_p, c_char_p, c_double, c_float

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libfpq_b200.so")

FPQ_OK = 0
FMT_MXFP4, FMT_NVFP4 = 0, 1
DT_BF16, DT_F32 = 0, 1
SCALES_ROWMAJOR, SCALES_SWIZZLED = 0, 1
OUT_CODES, OUT_GRID, OUT_DEQUANT, OUT_DEQUANT_STE = 0, 1, 2, 3
RELATIVE_MSE_ACC_DOUBLES = 32768
ERR_DEVICE_TIMEOUT = -4
ERR_NOT_POSITIVE_DEFINITE = -5

# name -> argument ctypes (all return int unless listed in _RESTYPES)
_SIGNATURES = {
    "fpq_version": [],
    "fpq_last_error": [],
    "fpq_check_device": [c_int],
    "fpq_rotate_hadamard": [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p],
    "fpq_rotate_dense": [c_void_p, c_int, c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p],
    "fpq_absmax": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p],
    "fpq_global_scale_update": [c_void_p, c_void_p, c_void_p, c_void_p],
    "fpq_quantize": [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p,
                     c_int, c_void_p, c_void_p],
    "fpq_quantize_silu_mul": [c_void_p, c_void_p, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "fpq_fake_quantize": [c_void_p, c_int, c_int64, c_int64, c_int, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "fpq_quantize_quest": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p, c_void_p],
    "fpq_fake_quantize_quest": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_void_p, c_void_p],
    "fpq_apply_scales": [c_void_p, c_int, c_int64, c_int64, c_void_p, c_int, c_int, c_void_p, c_void_p],
    "fpq_pack_grid": [c_void_p, c_int, c_int64, c_int64, c_void_p, c_void_p],
    "fpq_swizzle_scales": [c_void_p, c_int64, c_int64, c_void_p, c_void_p],
    "fpq_sgemm": [c_void_p, c_int64, c_void_p, c_int64, c_int, c_void_p, c_int64, c_int64, c_int64, c_int64,
                  c_float, c_float, c_void_p],
    "fpq_hessian_accumulate": [c_void_p, c_int64, c_void_p, c_void_p, c_int64, c_float, c_float, c_void_p, c_void_p],
    "fpq_hessian_prepare": [c_void_p, c_int64, c_void_p, c_int64, c_float, c_void_p, c_void_p],
    "fpq_hessian_prepare_noalloc": [c_void_p, c_int64, c_void_p, c_int64, c_float, c_void_p],
    "fpq_cholesky_workspace_floats": [c_int64],
    "fpq_cholesky_inverse_upper": [c_void_p, c_void_p, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    "fpq_gptq_quantize": [c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                          c_void_p],
    "fpq_mse_scales": [c_void_p, c_int, c_int64, c_int64, c_int, c_void_p, c_int, c_double, c_float, c_void_p, c_void_p],
    "fpq_gptq_quantize_ordered": [c_void_p, c_int64, c_int64, c_void_p, c_int, c_void_p, c_void_p, c_void_p, c_void_p,
                                  c_void_p, c_void_p],
    "fpq_gptq_workspace_bytes": [c_int64, c_int64],
    "fpq_relative_mse": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p],
    "fpq_relative_mse_tc": [c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                            c_void_p, c_void_p],
    "fpq_gemm_fp4_push": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_int64,
                          c_int64, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p],
    "fpq_gemm_fp4": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64,
                     c_int64, c_int, c_void_p, c_void_p],
    "fpq_quantize_mxfp8_square": [c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_void_p, c_void_p, c_int, c_void_p],
    "fpq_mxfp4_transpose_mxfp8": [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int, c_void_p],
    "fpq_mxfp4_transpose_dequant": [c_void_p, c_void_p, c_int64, c_int64, c_void_p, c_void_p, c_int64, c_void_p],
    "fpq_quantize_transposed": [c_void_p, c_int64, c_int64, c_int64, c_int, c_void_p, c_void_p, c_int, c_void_p],
    "fpq_gemm_mxf8": [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_int64, c_int64, c_int64,
                      c_void_p, c_void_p],
}
_RESTYPES = {"fpq_last_error": c_char_p, "fpq_cholesky_workspace_floats": c_int64,
             "fpq_gptq_workspace_bytes": c_int64}

_lib = None


class FpqError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"fpq_b200 status {status}: {message}")
        self.status = status


def exported_symbols():
    """Names every build of the library must export (mirrors include/fpq_b200.h)."""
    return sorted(_SIGNATURES)


def register(name: str, argtypes, restype=c_int):
    """Used by sibling modules to declare entry points added alongside new kernels."""
    _SIGNATURES[name] = argtypes
    if restype is not c_int:
        _RESTYPES[name] = restype
    if _lib is not None:
        fn = getattr(_lib, name)
        fn.argtypes = argtypes
        fn.restype = restype


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} not found: build it with `python -m fpq_b200._build` "
                "(needs nvcc 12.9; there is no CPU fallback)")
        _lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in _SIGNATURES.items():
            fn = getattr(_lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, c_int)
    return _lib


def check(status: int):
    if status != FPQ_OK:
        msg = lib().fpq_last_error()
        raise FpqError(status, msg.decode() if msg else "")


def call(name: str, *args):
    check(getattr(lib(), name)(*args))
