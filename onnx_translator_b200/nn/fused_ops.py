"""Graph nodes that stand for a chain of reference operators executed by one fused library call.
They are created by ``Graph.fused()``, never by a model import, and have the node interface of the
operator classes in Operators.py (``inputs``, ``outputs``, ``forward`` returning the result dict)."""
from __future__ import annotations

import ctypes

from . import Ops, Tensor
from .. import capi
from ..capi import CConvParams, CQConvCall
from ..device import DeviceArray
from .Operators import _int_ptr, _pooled_extent


def _conv_params(pads, strides, dilations):
    keep = [_int_ptr(pads), _int_ptr(strides), _int_ptr(dilations)]
    return CConvParams(keep[0][1], keep[1][1], keep[2][1], 1), keep


class QLinearConv(Ops):
    """DequantizeLinear(activation codes) + DequantizeLinear(weight codes) + Conv [+ Add(residual)] [+ Relu]
    in one call (replaces nn/Operators.py:452-473 twice, :475-548 and :170-200).

    inputs: [x, x_scale, x_zero, w_codes, w_scale, bias or "", residual or "", next_scale or "", next_zero or ""]

    * ``from_float``: x is the float32 tensor and the QuantizeLinear that makes the codes (:427-450) is part of
      the call; otherwise x holds the int8 / uint8 codes.
    * ``levels_in``: x is the levels tensor the producing QLinearConv wrote for this convolution.
    * ``next_conv`` (dict with pads, strides, dilations, kernel): the result is handed to the next quantised
      convolution as integer levels (quantised with next_scale / next_zero) instead of as float32 -- or, with
      ``also_float``, besides the float32 tensor (two outputs), when other nodes read the float32 values too.
    * ``x_channels_last`` / ``y_channels_last`` / ``residual_channels_last``: that float32 tensor is stored
      [N, H, W, C] instead of the ABI's NCHW.  ``Graph.fused()`` sets these on edges that only fused convolutions
      touch; such a ``Tensor`` carries ``channels_last = True`` and its NCHW shape in ``logical_shape``."""

    def __init__(self, inputs, outputs, pads, strides, dilations, relu, dtype="float32", from_float=False):
        super().__init__(inputs, outputs)
        self.pads, self.strides, self.dilations, self.relu, self.dtype = list(pads), list(strides), list(dilations), bool(relu), dtype
        self.from_float = bool(from_float)
        self.levels_in = False
        self.next_conv = None
        self.also_float = False       # with next_conv: outputs are (float32 tensor, levels tensor) instead of the levels alone
        self.x_channels_last = self.y_channels_last = self.residual_channels_last = False
        # The filters in the layout the tensor cores read, made by the library on the first call and reused while
        # the node keeps seeing the same weight array (replace the array, or call drop_filter_cache(), after
        # changing weights in place).
        self._filter_cache = ctypes.c_void_p()
        self._filter_cache_key = None

    def drop_filter_cache(self):
        if self._filter_cache:
            self.lib.free_tensor(ctypes.cast(self._filter_cache, capi.TensorP))
        self._filter_cache = ctypes.c_void_p()
        self._filter_cache_key = None

    def __del__(self):
        try:
            self.drop_filter_cache()
        except Exception:
            pass

    def _levels_tensor(self, logical_shape, conv):
        """bfloat16 levels tensor for the convolution described by ``conv`` reading ``logical_shape``."""
        params, keep = _conv_params(conv["pads"], conv["strides"], conv["dilations"])
        shape = (ctypes.c_int * 4)()
        rc = self.lib.tops_qconv_levels_shape((ctypes.c_int * 4)(*logical_shape), (ctypes.c_int * 2)(*conv["kernel"]),
                                              ctypes.byref(params), shape)
        if rc:
            capi.check(self.lib)
        # padding cells and padding channels are never written by the producer: they must read as zero
        n, c, h, w = logical_shape
        padded = tuple(shape) != (n, h, w, c)
        return DeviceArray.empty(tuple(shape), "bfloat16", zero=padded, lib=self.lib)

    def forward(self, x: Tensor, x_scale: Tensor, x_zero: Tensor, wq: Tensor, w_scale: Tensor, b: Tensor = None,
                residual: Tensor = None, next_scale: Tensor = None, next_zero: Tensor = None) -> dict:
        n, _, h, w = x.logical_shape if (self.levels_in or self.x_channels_last) else x.data.shape
        m, _, kh, kw = wq.data.shape
        out_shape = (n, m,
                     _pooled_extent(h, self.pads[0], self.pads[2], self.dilations[0], kh, self.strides[0]),
                     _pooled_extent(w, self.pads[1], self.pads[3], self.dilations[1], kw, self.strides[1]))
        if residual is not None and self.residual_channels_last and tuple(residual.logical_shape) != out_shape:
            raise ValueError(f"{self.name}: the channels-last residual has shape {residual.logical_shape}, the convolution gives {out_shape}")
        if residual is not None and not self.residual_channels_last and (tuple(residual.data.shape) != out_shape or residual.dtype != "float32"):
            # a broadcasting or converting Add is not what the fused epilogue does: run the three operators
            from .Operators import ADD, RELU
            plain = QLinearConv([], [], self.pads, self.strides, self.dilations, False, self.dtype, self.from_float)
            plain.levels_in, plain.x_channels_last = self.levels_in, self.x_channels_last
            y = ADD([], [], dtype=self.dtype).forward(plain.forward(x, x_scale, x_zero, wq, w_scale, b)["tensor"], residual)["tensor"]
            return self._publish(RELU([], [], dtype=self.dtype).forward(y)["tensor"] if self.relu else y)

        params, keep = _conv_params(self.pads, self.strides, self.dilations)
        operands = [t for t in (x, x_scale, x_zero, wq, w_scale, b, residual, next_scale, next_zero) if t is not None]
        handles = {id(t): self._numpy_to_ctensor(t.data, t.dtype) for t in operands}
        ptr = lambda t: None if t is None else ctypes.cast(handles[id(t)], ctypes.c_void_p)
        call = CQConvCall()
        call.x, call.x_levels = ptr(x), int(self.levels_in)
        if self.levels_in:
            call.x_shape = (ctypes.c_int * 4)(*x.logical_shape)
        call.x_scale, call.x_zero, call.w_codes, call.w_scale = ptr(x_scale), ptr(x_zero), ptr(wq), ptr(w_scale)
        call.bias, call.residual = ptr(b), ptr(residual)
        call.x_channels_last, call.residual_channels_last = int(self.x_channels_last), int(self.residual_channels_last and residual is not None)
        call.params, call.relu = ctypes.pointer(params), int(self.relu)
        key = (id(wq.data), tuple(wq.data.shape), bool(self.levels_in), tuple(self.pads), tuple(self.strides), tuple(self.dilations))
        if key != self._filter_cache_key:
            self.drop_filter_cache()
            self._filter_cache_key = key
        call.filter_cache = ctypes.pointer(self._filter_cache)
        y_handle = levels = None
        if self.next_conv is not None:
            levels = self._levels_tensor(out_shape, self.next_conv)
            next_params, keep_next = _conv_params(self.next_conv["pads"], self.next_conv["strides"], self.next_conv["dilations"])
            call.y_levels = ctypes.cast(levels.handle, ctypes.c_void_p)
            call.next_scale, call.next_zero = ptr(next_scale), ptr(next_zero)
            call.next_params = ctypes.pointer(next_params)
            call.next_kernel = (ctypes.c_int * 2)(*self.next_conv["kernel"])
        stored_shape = (out_shape[0], out_shape[2], out_shape[3], out_shape[1]) if self.y_channels_last else out_shape
        if self.next_conv is None or self.also_float:
            y_handle = self._new_output(stored_shape, self.dtype)
            call.y, call.y_channels_last = ctypes.cast(y_handle, ctypes.c_void_p), int(self.y_channels_last)
        rc = self.lib.tops_qconv_forward(ctypes.byref(call))
        for hdl in handles.values():
            self.lib.free_tensor(hdl)
        if rc:
            if y_handle is not None:
                self.lib.free_tensor(y_handle)
            capi.check(self.lib)
        result = None if y_handle is None else self._finish([], y_handle, stored_shape, self.dtype)
        if result is not None and self.y_channels_last:
            result.channels_last, result.logical_shape = True, out_shape
        if levels is not None:
            out = Tensor(*levels.shape, dtype="bfloat16", data=levels)
            out.logical_shape = out_shape
            result = out if result is None else (result, out)
        return self._publish(result)


class QuantizeDequantize(Ops):
    """QuantizeLinear followed by DequantizeLinear with the same scale and zero point, in one pass over the tensor
    (replaces nn/Operators.py:427-450 and :452-473; C: tensor_ops.c:999-1034).  ``outputs`` is [dequantised] or
    [dequantised, codes] when something else reads the codes.  Falls back to the two operators for what the fused
    call does not cover (other dtypes than float32, broadcast patterns it cannot collapse)."""

    def __init__(self, inputs, outputs, axis=1, code_dtype="int8", dtype="float32", with_codes=False):
        super().__init__(inputs, outputs)
        self.axis, self.code_dtype, self.dtype, self.with_codes = axis, code_dtype, dtype, bool(with_codes)

    def _two_operators(self, x, scale, zero):
        from .Operators import DequantizeLinear, QuantizeLinear
        codes = QuantizeLinear([], [], axis=self.axis, dtype=self.code_dtype).forward(x, scale, zero)["tensor"]
        s, z = scale, zero
        if scale.data.ndim == 1 and x.data.ndim > 1:         # DequantizeLinear has no axis: hand it the reshaped operands
            shape = [1] * x.data.ndim
            shape[self.axis if self.axis >= 0 else self.axis + x.data.ndim] = scale.data.size
            s = Tensor(*shape, dtype=scale.dtype, data=scale.data.reshape(shape))
            z = Tensor(*shape, dtype=zero.dtype, data=zero.data.reshape(shape))
        y = DequantizeLinear([], [], dtype=self.dtype).forward(codes, s, z)["tensor"]
        return self._publish((y, codes) if self.with_codes else y)

    def forward(self, x: Tensor, scale: Tensor, zero: Tensor) -> dict:
        if x.dtype != "float32" or self.dtype != "float32" or scale.dtype != "float32":
            return self._two_operators(x, scale, zero)
        shape = tuple(x.data.shape)
        s_data, z_data = scale.data, zero.data
        if s_data.ndim == 1 and len(shape) > 1:                # a 1-D scale sits on ``axis`` (nn/Operators.py:439-445)
            bshape = [1] * len(shape)
            bshape[self.axis if self.axis >= 0 else self.axis + len(shape)] = s_data.size
            s_data, z_data = s_data.reshape(bshape), z_data.reshape(bshape)
        handles = [self._numpy_to_ctensor(x.data, x.dtype), self._numpy_to_ctensor(s_data, scale.dtype), self._numpy_to_ctensor(z_data, zero.dtype)]
        y = self._new_output(shape, "float32")
        codes = self._new_output(shape, self.code_dtype) if self.with_codes else None
        rc = self.lib.tops_quantize_dequantize_forward(handles[0], handles[1], handles[2], codes, y)
        if rc:
            for h in handles + [y] + ([codes] if codes else []):
                self.lib.free_tensor(h)
            code = self.lib.tops_last_error()
            self.lib.tops_clear_error()
            if code != 5:                                       # anything but "unsupported" is a real error
                raise capi.TensorOpsError(f"tops_quantize_dequantize_forward failed with code {code}")
            return self._two_operators(x, scale, zero)
        code_tensor = self._finish([], codes, shape, self.code_dtype) if codes else None
        out = self._finish(handles, y, shape, "float32")
        return self._publish((out, code_tensor) if self.with_codes else out)


class DequantAddQuant(Ops):
    """QuantizeLinear([Relu](DequantizeLinear(a) + DequantizeLinear(b))) in one pass: the tail of a quantised
    residual block (replaces nn/Operators.py:452-473 twice, :170-200, :32-80 and :427-450).
    inputs: [a, a_scale, a_zero, b, b_scale, b_zero, y_scale, y_zero]."""

    def __init__(self, inputs, outputs, relu=False, dtype="int8"):
        super().__init__(inputs, outputs)
        self.relu, self.dtype = bool(relu), dtype

    def _five_operators(self, a, a_s, a_z, b, b_s, b_z, y_s, y_z):
        from .Operators import ADD, RELU, DequantizeLinear, QuantizeLinear
        da = DequantizeLinear([], [], dtype="float32").forward(a, a_s, a_z)["tensor"]
        db = DequantizeLinear([], [], dtype="float32").forward(b, b_s, b_z)["tensor"]
        t = ADD([], [], dtype="float32").forward(da, db)["tensor"]
        if self.relu:
            t = RELU([], [], dtype="float32").forward(t)["tensor"]
        return self._publish(QuantizeLinear([], [], axis=1, dtype=self.dtype).forward(t, y_s, y_z)["tensor"])

    def forward(self, a, a_s, a_z, b, b_s, b_z, y_s, y_z) -> dict:
        shape = tuple(a.data.shape)
        if tuple(b.data.shape) != shape:
            return self._five_operators(a, a_s, a_z, b, b_s, b_z, y_s, y_z)
        operands = (a, a_s, a_z, b, b_s, b_z, y_s, y_z)
        handles = [self._numpy_to_ctensor(t.data, t.dtype) for t in operands]
        y = self._new_output(shape, self.dtype)
        rc = self.lib.tops_dq_add_q_forward(*handles, y, int(self.relu))
        if rc:
            for h in handles + [y]:
                self.lib.free_tensor(h)
            code = self.lib.tops_last_error()
            self.lib.tops_clear_error()
            if code != 5:
                raise capi.TensorOpsError(f"tops_dq_add_q_forward failed with code {code}")
            return self._five_operators(*operands)
        return self._publish(self._finish(handles, y, shape, self.dtype))
