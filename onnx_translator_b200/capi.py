"""ctypes binding of the operator library (``lib/tensor_ops.so``).

This is the only place the shared object is opened.  There is no fallback of any kind: if the
library has not been built, or the machine has no CUDA device, loading or the first call fails
with an error that says so.

The structures and tables mirror the reference's Python side (nn/__init__.py:9-72,
nn/Operators.py:9-23) so that its operator classes can drive this library unchanged.
"""
from __future__ import annotations

import ctypes
import os
from typing import Optional

import numpy as np

PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(PKG, "lib", "tensor_ops.so")


class CTensor(ctypes.Structure):
    """struct Tensor of include/tensor_ops_b200.h (tensor_ops/tensor_ops.h:28-34)."""
    _fields_ = [("data", ctypes.c_void_p),
                ("shape", ctypes.POINTER(ctypes.c_int)),
                ("ndim", ctypes.c_int),
                ("size", ctypes.c_size_t),
                ("dtype", ctypes.c_int)]


class CConvParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("group", ctypes.c_int)]


class CQConvCall(ctypes.Structure):
    """QConvCall of tensor_ops_b200.h."""
    _fields_ = [("x", ctypes.c_void_p), ("x_levels", ctypes.c_int), ("x_shape", ctypes.c_int * 4),
                ("x_scale", ctypes.c_void_p), ("x_zero", ctypes.c_void_p), ("w_codes", ctypes.c_void_p), ("w_scale", ctypes.c_void_p),
                ("bias", ctypes.c_void_p), ("residual", ctypes.c_void_p), ("params", ctypes.POINTER(CConvParams)), ("relu", ctypes.c_int),
                ("y", ctypes.c_void_p), ("y_levels", ctypes.c_void_p), ("next_scale", ctypes.c_void_p), ("next_zero", ctypes.c_void_p),
                ("next_params", ctypes.POINTER(CConvParams)), ("next_kernel", ctypes.c_int * 2),
                ("filter_cache", ctypes.POINTER(ctypes.c_void_p)),
                ("x_channels_last", ctypes.c_int), ("y_channels_last", ctypes.c_int), ("residual_channels_last", ctypes.c_int)]


class CPoolParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("kernel_shape", ctypes.POINTER(ctypes.c_int))]


TensorP = ctypes.POINTER(CTensor)

# dtype name -> enum code (nn/__init__.py:20-34); "bool" shares uint8's code there too
DTYPE_MAP = {
    "float8_e4m3": 0, "float8_e5m2": 1, "float16": 2, "bfloat16": 3, "float32": 4, "float64": 5,
    "int4": 6, "int8": 7, "uint8": 8, "int16": 9, "int32": 10, "int64": 11, "bool": 8,
}
CODE_TO_DTYPE = {v: k for k, v in DTYPE_MAP.items() if k != "bool"}

# host storage per dtype (nn/__init__.py:37-51): fp8 as uint8 codes, bfloat16 as uint16 codes
DTYPE_TO_NUMPY = {
    "float8_e4m3": np.uint8, "float8_e5m2": np.uint8, "float16": np.float16, "bfloat16": np.uint16,
    "float32": np.float32, "float64": np.float64, "int4": np.int8, "int8": np.int8, "uint8": np.uint8,
    "int16": np.int16, "int32": np.int32, "int64": np.int64, "bool": np.bool_,
}

# numpy scalar type -> dtype name used for output-type inference (nn/__init__.py:54-72)
NUMPY_TO_DTYPE = {
    np.float16: "float16", np.uint16: "bfloat16", np.float32: "float32", np.float64: "float64",
    np.int8: "int8", np.uint8: "uint8", np.int16: "int16", np.int32: "int32", np.int64: "int64",
    np.uint32: "uint32", np.uint64: "uint64",
}

ERROR_NAMES = {0: "ok", 1: "invalid argument", 2: "CUDA error", 3: "no CUDA device", 4: "out of memory",
               5: "unsupported", 6: "device-side wait timed out"}


class TensorOpsError(RuntimeError):
    pass


# name -> (restype, argtypes); every symbol declared in include/tensor_ops_b200.h
_P, _I, _F, _V, _SZ = TensorP, ctypes.c_int, ctypes.c_float, ctypes.c_void_p, ctypes.c_size_t
_IP = ctypes.POINTER(ctypes.c_int)
SIGNATURES = {
    # reference entry points
    "create_tensor": (_P, [_IP, _I, _I]),
    "free_tensor": (None, [_P]),
    "init_cos_lut": (None, []),
    "relu_forward": (None, [_P, _P]),
    "cos_forward": (None, [_P, _P]),
    "abs_forward": (None, [_P, _P]),
    "add_forward": (None, [_P, _P, _P]),
    "sub_forward": (None, [_P, _P, _P]),
    "mul_forward": (None, [_P, _P, _P]),
    "div_forward": (None, [_P, _P, _P]),
    "quantize_linear_forward": (None, [_P, _P, _P, _P]),
    "dequantize_linear_forward": (None, [_P, _P, _P, _P]),
    "conv2d_forward": (None, [_P, _P, _P, _P, ctypes.POINTER(CConvParams)]),
    "max_pool_forward": (None, [_P, _P, ctypes.POINTER(CPoolParams)]),
    "gemm_forward": (None, [_P, _P, _P, _P, _F, _F, _I, _I]),
    "softmax_forward": (None, [_P, _P, _I]),
    "flatten_forward": (None, [_P, _P]),
    "reshape_forward": (None, [_P, _P]),
    # additive interface
    "tops_last_error": (_I, []),
    "tops_last_error_message": (ctypes.c_char_p, []),
    "tops_clear_error": (None, []),
    "tops_set_device": (_I, [_I]),
    "tops_get_device": (_I, []),
    "tops_device_count": (_I, []),
    "tops_get_stream": (_V, []),
    "tops_set_stream": (_I, [_V]),
    "tops_sync": (_I, []),
    "tops_set_memory_mode": (_I, [_I]),
    "tops_capture_begin": (_I, []),
    "tops_capture_end": (_V, []),
    "tops_capture_launch": (_I, [_V]),
    "tops_capture_free": (None, [_V]),
    "tops_create_uninit": (_P, [_IP, _I, _I]),
    "tops_wrap": (_P, [_V, _IP, _I, _I]),
    "tops_view": (_P, [_P, _IP, _I]),
    "tops_slice_rows": (_P, [_P, _I, _I]),
    "tops_retain": (None, [_P]),
    "tops_upload": (_I, [_P, _V, _SZ]),
    "tops_download": (_I, [_P, _V, _SZ]),
    "tops_download_async": (_I, [_P, _V, _SZ]),
    "tops_host_alloc": (_V, [_SZ]),
    "tops_host_free": (None, [_V]),
    "tops_dtype_size": (_SZ, [_I]),
    "cast_forward": (None, [_P, _P]),
    "max_forward": (None, [_P, _P, _P]),
    "min_forward": (None, [_P, _P, _P]),
    "pow_forward": (None, [_P, _P, _P]),
    **{name + "_forward": (None, [_P, _P]) for name in (
        "exp", "log", "sqrt", "sigmoid", "tanh", "neg", "reciprocal", "ceil", "floor", "sin", "tan", "atan", "softplus", "softsign",
        "hard_swish", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "round", "erf", "gelu")},
    "clip_forward": (None, [_P, _P, _P, _P]),
    "average_pool_forward": (None, [_P, _P, ctypes.POINTER(CPoolParams), _I]),
    "global_average_pool_forward": (None, [_P, _P]),
    "batch_norm_forward": (None, [_P, _P, _P, _P, _P, _P, ctypes.c_float]),
    "matmul_forward": (None, [_P, _P, _P]),
    "dynamic_quantize_linear_forward": (None, [_P, _P, _P, _P]),
    "tops_dynamic_quantize_range": (ctypes.c_int, [_P, _P]),
    "tops_dynamic_quantize_apply": (ctypes.c_int, [_P, _P, _P, _P, _P]),
    "tops_quantize_linear_axis_forward": (None, [_P, _P, _P, _P, _I]),
    "tops_dequantize_linear_axis_forward": (None, [_P, _P, _P, _P, _I]),
    "tops_quantize_dequantize_forward": (_I, [_P, _P, _P, _P, _P]),
    "tops_dq_add_q_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I]),
    "tops_conv2d_forward_noalloc": (None, [_P, _P, _P, _P, ctypes.POINTER(CConvParams)]),
    "tops_conv2d_noalloc_prepare": (_I, []),
    "tops_conv2d_noalloc_limits": (_SZ, [ctypes.POINTER(_SZ), ctypes.POINTER(_SZ)]),
    "tops_gemm_qdq_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, ctypes.c_float, ctypes.c_float, _I, _I]),
    "tops_conv2d_dqw_forward": (_I, [_P, _P, _P, _P, _P, ctypes.POINTER(CConvParams)]),
    "tops_qlinear_conv_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, ctypes.POINTER(CConvParams), _I]),
    "tops_qdq_conv_forward": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, ctypes.POINTER(CConvParams), _I]),
    "tops_qconv_forward": (_I, [ctypes.POINTER(CQConvCall)]),
    "tops_qconv_levels_shape": (_I, [ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int), ctypes.POINTER(CConvParams),
                                     ctypes.POINTER(ctypes.c_int)]),
    "tops_selftest_encoder": (ctypes.c_longlong, [_I]),
    "tops_tensor_core_launches": (ctypes.c_longlong, []),
    "tops_selftest_cos": (ctypes.c_longlong, []),
    "tops_selftest_wait_timeout": (_I, [_I]),
    "tops_debug_plan_broadcast": (_I, [_IP, _I, _IP, _I, _IP, ctypes.POINTER(ctypes.c_uint), _IP, _IP]),
    "tops_version": (ctypes.c_char_p, []),
}

_lib: Optional[ctypes.CDLL] = None


def load(path: Optional[str] = None) -> ctypes.CDLL:
    """Open the shared object and declare every signature.  Raises if it is not built."""
    global _lib
    if _lib is not None and path is None:
        return _lib
    path = path or os.environ.get("TENSOR_OPS_B200_LIB") or LIB_PATH
    if not os.path.exists(path):
        raise TensorOpsError(
            f"{path} is missing: build it with `python -m onnx_translator_b200.build` "
            "(there is no CPU fallback)")
    lib = ctypes.CDLL(path)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)          # AttributeError here means header and library disagree
        fn.restype = restype
        fn.argtypes = argtypes
    if path == LIB_PATH or _lib is None:
        _lib = lib
    return lib


def check(lib: Optional[ctypes.CDLL] = None) -> None:
    """Raise TensorOpsError if the library has recorded an error, then clear it."""
    lib = lib or load()
    code = lib.tops_last_error()
    if code:
        msg = lib.tops_last_error_message().decode(errors="replace")
        lib.tops_clear_error()
        raise TensorOpsError(f"{ERROR_NAMES.get(code, code)}: {msg}")


def shape_array(shape):
    shape = tuple(int(s) for s in shape)
    return (ctypes.c_int * max(len(shape), 1))(*shape), len(shape)
