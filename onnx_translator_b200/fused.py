"""Host side of the fused entry points: the operator chains of quantised graphs in one call.

``gemm_qdq`` stands for DequantizeLinear(A), DequantizeLinear(B) -> Gemm -> [QuantizeLinear] and
``conv2d_dqw`` for DequantizeLinear(W, per output channel) -> Conv, i.e. for chains of the operator
classes in nn/Operators.py (reference: nn/Operators.py:427-473, 475-548, 613-669).  Operands and
results are device-resident ``DeviceArray`` objects; nothing is copied to the host.  A case the
fused kernels do not cover raises ``TensorOpsError`` (the unfused chain of operators covers it).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import capi
from .capi import CConvParams
from .device import DeviceArray


def _as_device(x, dtype_name: Optional[str] = None) -> DeviceArray:
    return x if isinstance(x, DeviceArray) else DeviceArray.from_numpy(np.asarray(x), dtype_name)


def _scale(x) -> DeviceArray:
    if isinstance(x, DeviceArray):
        return x
    return DeviceArray.from_numpy(np.atleast_1d(np.asarray(x, dtype=np.float32)), "float32")


def gemm_qdq(a, a_scale, b, b_scale, c=None, y_scale=None, out_dtype: str = "float32",
             alpha: float = 1.0, beta: float = 1.0, a_dtype: str = "float8_e4m3", b_dtype: str = "float8_e4m3") -> DeviceArray:
    """Y = [Q]( alpha * DQ(A, a_scale) @ DQ(B, b_scale).T + beta * C ).  A is [M, K], B is [N, K],
    both fp8 codes; with ``y_scale`` the result is quantised to ``out_dtype`` (an 8-bit type)."""
    lib = capi.load()
    a, b = _as_device(a, a_dtype), _as_device(b, b_dtype)
    sa, sb = _scale(a_scale), _scale(b_scale)
    sy = None if y_scale is None else _scale(y_scale)
    cc = None if c is None else _as_device(c, "float32")
    y = DeviceArray.empty((a.shape[0], b.shape[0]), out_dtype, lib=lib)
    rc = lib.tops_gemm_qdq_forward(a.handle, sa.handle, b.handle, sb.handle, cc.handle if cc is not None else None,
                                   sy.handle if sy is not None else None, y.handle,
                                   ctypes.c_float(alpha), ctypes.c_float(beta), 0, 1)
    if rc:
        capi.check(lib)
    return y


def conv2d_dqw(x, wq, w_scale, bias=None, out_dtype: str = "float32", pads: Sequence[int] = (0, 0, 0, 0),
               dilations: Sequence[int] = (1, 1), x_dtype: str = "bfloat16") -> DeviceArray:
    """Y = Conv(X, DQ(Wq, w_scale per output channel), bias), stride 1, group 1.  X is NCHW float16 or
    bfloat16, Wq is [M, C, KH, KW] int8 codes, w_scale is [M] float32."""
    lib = capi.load()
    x = _as_device(x, x_dtype)
    wq = _as_device(wq, "int8")
    ws = _scale(w_scale)
    bb = None if bias is None else _as_device(bias, "float32")
    n, _, h, w = x.shape
    m, _, kh, kw = wq.shape
    oh = h + pads[0] + pads[2] - dilations[0] * (kh - 1)
    ow = w + pads[1] + pads[3] - dilations[1] * (kw - 1)
    y = DeviceArray.empty((n, m, oh, ow), out_dtype, lib=lib)
    keep = [(ctypes.c_int * 4)(*pads), (ctypes.c_int * 2)(1, 1), (ctypes.c_int * 2)(*dilations)]
    params = CConvParams(keep[0], keep[1], keep[2], 1)
    rc = lib.tops_conv2d_dqw_forward(x.handle, wq.handle, ws.handle, bb.handle if bb is not None else None, y.handle,
                                     ctypes.byref(params))
    if rc:
        capi.check(lib)
    return y
