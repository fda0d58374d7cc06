"""Graph nodes that stand for a chain of reference operators executed by one fused library call.
They are created by ``Graph.fused()``, never by a model import, and have the node interface of the
operator classes in Operators.py (``inputs``, ``outputs``, ``forward`` returning the result dict)."""
from __future__ import annotations

import ctypes

from . import Ops, Tensor
from .. import capi
from ..capi import CConvParams
from .Operators import _int_ptr, _pooled_extent


class QLinearConv(Ops):
    """DequantizeLinear(activation codes) + DequantizeLinear(weight codes) + Conv [+ Relu] in one call
    (replaces nn/Operators.py:452-473 twice, :475-548 and :170-200).
    inputs: [x_codes, x_scale, x_zero, w_codes, w_scale, bias or "", residual or ""]; a residual is a float32
    tensor of the output's shape that is added before the optional Relu (the Add node :170-200 of a
    residual block).  With ``from_float`` the first input
    is the float32 tensor and the QuantizeLinear that makes the codes (:427-450) is part of the call too."""

    def __init__(self, inputs, outputs, pads, strides, dilations, relu, dtype="float32", from_float=False):
        super().__init__(inputs, outputs)
        self.pads, self.strides, self.dilations, self.relu, self.dtype = list(pads), list(strides), list(dilations), bool(relu), dtype
        self.from_float = bool(from_float)

    def forward(self, xq: Tensor, x_scale: Tensor, x_zero: Tensor, wq: Tensor, w_scale: Tensor, b: Tensor = None,
                residual: Tensor = None) -> dict:
        n, _, h, w = xq.data.shape
        m, _, kh, kw = wq.data.shape
        out_shape = (n, m,
                     _pooled_extent(h, self.pads[0], self.pads[2], self.dilations[0], kh, self.strides[0]),
                     _pooled_extent(w, self.pads[1], self.pads[3], self.dilations[1], kw, self.strides[1]))
        if residual is not None and tuple(residual.data.shape) != out_shape:
            # a broadcasting Add is not what the fused epilogue does: run the three operators
            from .Operators import ADD, RELU
            plain = QLinearConv([], [], self.pads, self.strides, self.dilations, False, self.dtype, self.from_float)
            y = ADD([], [], dtype=self.dtype).forward(plain.forward(xq, x_scale, x_zero, wq, w_scale, b)["tensor"], residual)["tensor"]
            return self._publish(RELU([], [], dtype=self.dtype).forward(y)["tensor"] if self.relu else y)
        keep = [_int_ptr(self.pads), _int_ptr(self.strides), _int_ptr(self.dilations)]
        params = CConvParams(keep[0][1], keep[1][1], keep[2][1], 1)
        operands = [xq, x_scale, x_zero, wq, w_scale] + [t for t in (b, residual) if t is not None]
        handles = [self._numpy_to_ctensor(t.data, t.dtype) for t in operands]
        b_handle = handles[5] if b is not None else None
        r_handle = handles[-1] if residual is not None else None
        y = self._new_output(out_shape, self.dtype)
        entry = self.lib.tops_qdq_conv_forward if self.from_float else self.lib.tops_qlinear_conv_forward
        rc = entry(handles[0], handles[1], handles[2], handles[3], handles[4], b_handle, r_handle, y,
                   ctypes.byref(params), int(self.relu))
        out = self._finish(handles, y, out_shape, self.dtype) if not rc else None
        if rc:
            for hdl in handles:
                self.lib.free_tensor(hdl)
            self.lib.free_tensor(y)
            capi.check(self.lib)
        return self._publish(out)
