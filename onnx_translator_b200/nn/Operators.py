"""Operator classes of the hot path, with the reference's names, constructor signatures and
return convention (nn/Operators.py:32-818): ``forward`` computes on the GPU and returns
``{"tensor": Tensor, "parameters": None, "graph": None}``; ``forward_`` is the shape/dtype-only pass
over ``Tensor_`` placeholders.  Shape inference and attribute packing follow the reference; data
stay on the device (see ``nn.Ops``).
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import Ops, Tensor, Tensor_, DTYPE_MAP, DTYPE_TO_NUMPY, NUMPY_TO_DTYPE
from .. import capi
from ..capi import CConvParams, CPoolParams
from ..device import DeviceArray


def _int_ptr(values):
    arr = (ctypes.c_int * len(values))(*[int(v) for v in values])
    return arr, ctypes.cast(arr, ctypes.POINTER(ctypes.c_int))


def _pooled_extent(size, pad_a, pad_b, dilation, kernel, stride):
    return (size + pad_a + pad_b - dilation * (kernel - 1) - 1) // stride + 1


# ---- unary -----------------------------------------------------------------------------------------
class _Unary(Ops):
    _c_name = None

    def __init__(self, inputs, outputs, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype
        self.version = version

    def forward(self, input: Tensor) -> dict:
        return self._publish(self._execute_unary(input, self._c_name))

    def forward_(self, input: Tensor_) -> dict:
        return self._publish(Tensor_(*input.size, dtype=self.dtype))


class RELU(_Unary):
    """max(x, 0); integer inputs stay integer (nn/Operators.py:32-80)."""
    _c_name = "relu_forward"


class COS(_Unary):
    """Table cosine of the reference (nn/Operators.py:82-130)."""
    _c_name = "cos_forward"


class ABS(_Unary):
    """|x| (nn/Operators.py:132-168)."""
    _c_name = "abs_forward"


# ---- binary with broadcasting ------------------------------------------------------------------------
class _Binary(Ops):
    _c_name = None
    _label = None

    def __init__(self, inputs, outputs, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype                   # output dtype from the graph; None -> numpy promotion
        self.version = version

    def forward(self, *inputs) -> dict:
        if len(inputs) != 2:
            raise ValueError(f"{self._label} operator expects 2 inputs, but got {len(inputs)}")
        return self._publish(self._execute_binary(inputs[0], inputs[1], self._c_name))

    def forward_(self, *inputs) -> dict:
        if len(inputs) != 2:
            raise ValueError(f"{self._label} operator expects 2 inputs (Tensor_), but got {len(inputs)}")
        a, b = inputs
        try:
            shape = np.broadcast_shapes(tuple(a.size), tuple(b.size))
        except ValueError:
            print(f"Error during broadcasting shapes {a.size} and {b.size}")
            raise
        res = np.result_type(DTYPE_TO_NUMPY[a.dtype], DTYPE_TO_NUMPY[b.dtype])
        if res.type in NUMPY_TO_DTYPE:
            name = NUMPY_TO_DTYPE[res.type]
        elif "float" in str(res):
            name = "float64"
        elif "int" in str(res):
            name = "int64"
        else:
            name = "float32"
        return self._publish(Tensor_(*shape, dtype=name))


class ADD(_Binary):
    _c_name, _label = "add_forward", "ADD"


class SUB(_Binary):
    _c_name, _label = "sub_forward", "SUB"


class MUL(_Binary):
    _c_name, _label = "mul_forward", "MUL"


class DIV(_Binary):
    _c_name, _label = "div_forward", "DIV"


# ---- quantisation -------------------------------------------------------------------------------------
class QuantizeLinear(Ops):
    """y = saturate(rint(x / scale) + zero_point) (nn/Operators.py:427-450).  A 1-D scale on an
    N-D input is placed on ``axis``."""

    def __init__(self, inputs, outputs, axis=1, dtype=None, version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype
        self.axis = axis
        self.version = version

    def forward(self, x, y_scale, y_zero_point) -> dict:
        scale, zp = y_scale, y_zero_point
        if y_scale.data.ndim == 1 and x.data.ndim > 1:
            shape = [1] * x.data.ndim
            axis = self.axis if self.axis >= 0 else self.axis + x.data.ndim
            if axis < x.data.ndim:
                shape[axis] = y_scale.data.size
            scale = Tensor(*shape, dtype=y_scale.dtype, data=y_scale.data.reshape(shape))
            zp = Tensor(*shape, dtype=y_zero_point.dtype, data=y_zero_point.data.reshape(shape))
        return self._publish(self._execute_ternary(x, scale, zp, "quantize_linear_forward"))


class DequantizeLinear(Ops):
    """y = (x - zero_point) * scale with plain trailing-dimension broadcasting; there is no axis
    attribute (nn/Operators.py:452-473)."""

    def __init__(self, inputs, outputs, dtype=None, version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype
        self.version = version

    def forward(self, x, x_scale, x_zero_point) -> dict:
        return self._publish(self._execute_ternary(x, x_scale, x_zero_point, "dequantize_linear_forward"))

    def forward_(self, x, x_scale, x_zero_point) -> dict:
        try:
            shape = np.broadcast_shapes(tuple(x.size), tuple(x_scale.size), tuple(x_zero_point.size))
        except Exception:
            shape = x.size
        return self._publish(Tensor_(*shape, dtype=self.dtype))


# ---- structured operators ---------------------------------------------------------------------------------
class Conv(Ops):
    """2-D convolution over NCHW (nn/Operators.py:475-548).  pads = [top, left, bottom, right]."""

    def __init__(self, inputs, outputs, pads, strides, dilations, group, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.pads, self.strides, self.dilations, self.group = pads, strides, dilations, group
        self.dtype = dtype
        self.version = version

    def _out_shape(self, x_size, w_size):
        n, _, h, w = x_size
        m, _, kh, kw = w_size
        return (n, m,
                _pooled_extent(h, self.pads[0], self.pads[2], self.dilations[0], kh, self.strides[0]),
                _pooled_extent(w, self.pads[1], self.pads[3], self.dilations[1], kw, self.strides[1]))

    def forward(self, x: Tensor, w: Tensor, b: Tensor = None) -> dict:
        out_shape = self._out_shape(x.data.shape, w.data.shape)
        keep = [_int_ptr(self.pads), _int_ptr(self.strides), _int_ptr(self.dilations)]
        params = CConvParams(keep[0][1], keep[1][1], keep[2][1], int(self.group))
        handles = [self._numpy_to_ctensor(x.data, x.dtype), self._numpy_to_ctensor(w.data, w.dtype)]
        bias = None
        if b is not None:
            bias = self._numpy_to_ctensor(b.data, b.dtype)
            handles.append(bias)
        y = self._new_output(out_shape, self.dtype)
        self.lib.conv2d_forward(handles[0], handles[1], bias, y, ctypes.byref(params))
        return self._publish(self._finish(handles, y, out_shape, self.dtype))

    def forward_(self, x: Tensor_, w: Tensor_, b: Tensor_ = None) -> dict:
        return self._publish(Tensor_(*self._out_shape(x.size, w.size), dtype=self.dtype))


class MaxPool(Ops):
    """Max pooling over NCHW (nn/Operators.py:550-611)."""

    def __init__(self, inputs, outputs, kernel_shape, pads, strides, dtype, dilations=[1, 1], version="17"):
        super().__init__(inputs, outputs)
        self.kernel_shape, self.pads, self.strides, self.dilations = kernel_shape, pads, strides, dilations
        self.dtype = dtype
        self.version = version

    def forward(self, x: Tensor) -> dict:
        n, c, h, w = x.data.shape
        out_shape = (n, c,
                     _pooled_extent(h, self.pads[0], self.pads[2], self.dilations[0], self.kernel_shape[0], self.strides[0]),
                     _pooled_extent(w, self.pads[1], self.pads[3], self.dilations[1], self.kernel_shape[1], self.strides[1]))
        keep = [_int_ptr(self.pads), _int_ptr(self.strides), _int_ptr(self.dilations), _int_ptr(self.kernel_shape)]
        params = CPoolParams(keep[0][1], keep[1][1], keep[2][1], keep[3][1])
        xh = self._numpy_to_ctensor(x.data, x.dtype)
        y = self._new_output(out_shape, self.dtype)
        self.lib.max_pool_forward(xh, y, ctypes.byref(params))
        return self._publish(self._finish([xh], y, out_shape, self.dtype))

    def forward_(self, x: Tensor_) -> dict:
        # the reference's shape pass leaves dilation out (nn/Operators.py:606-607)
        n, c, h, w = x.size
        oh = (h + self.pads[0] + self.pads[2] - self.kernel_shape[0]) // self.strides[0] + 1
        ow = (w + self.pads[1] + self.pads[3] - self.kernel_shape[1]) // self.strides[1] + 1
        return self._publish(Tensor_(n, c, oh, ow, dtype=self.dtype))


class Gemm(Ops):
    """Y = alpha * A' B' + beta * C (nn/Operators.py:613-669).  A 1-D C is presented to the
    library as (1, N) when its length is N, else as (M, 1) when its length is M."""

    def __init__(self, inputs, outputs, alpha, beta, transA, transB, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.alpha, self.beta, self.transA, self.transB = alpha, beta, transA, transB
        self.dtype = dtype

    def _mn(self, a_size, b_size):
        m = a_size[0] if self.transA == 0 else a_size[1]
        n = b_size[1] if self.transB == 0 else b_size[0]
        return m, n

    def forward(self, A: Tensor, B: Tensor, C: Tensor = None) -> dict:
        m, n = self._mn(A.data.shape, B.data.shape)
        handles = [self._numpy_to_ctensor(A.data, A.dtype), self._numpy_to_ctensor(B.data, B.dtype)]
        c_handle = None
        if C is not None:
            c_data = C.data
            if c_data.ndim == 1:
                if c_data.shape[0] == n:
                    c_data = c_data.reshape(1, -1)
                elif c_data.shape[0] == m:
                    c_data = c_data.reshape(-1, 1)
            c_handle = self._numpy_to_ctensor(c_data, C.dtype)
            handles.append(c_handle)
        y = self._new_output((m, n), self.dtype)
        self.lib.gemm_forward(handles[0], handles[1], c_handle, y, float(self.alpha), float(self.beta),
                              int(self.transA), int(self.transB))
        return self._publish(self._finish(handles, y, (m, n), self.dtype))

    def forward_(self, A: Tensor_, B: Tensor_, C: Tensor_ = None) -> dict:
        return self._publish(Tensor_(*self._mn(A.size, B.size), dtype=self.dtype))


class Softmax(Ops):
    """Softmax along ``axis`` (nn/Operators.py:671-704)."""

    def __init__(self, inputs, outputs, axis, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.axis = axis
        self.dtype = dtype

    def forward(self, input: Tensor) -> dict:
        shape = tuple(input.data.shape)
        x = self._numpy_to_ctensor(input.data, input.dtype)
        y = self._new_output(shape, self.dtype)
        self.lib.softmax_forward(x, y, int(self.axis))
        return self._publish(self._finish([x], y, shape, self.dtype))

    def forward_(self, input: Tensor_) -> dict:
        return self._publish(Tensor_(*input.size, dtype=self.dtype))


class Flatten(Ops):
    """Reshape to [prod(shape[:axis]), prod(shape[axis:])] (nn/Operators.py:776-818).  On the
    device this is a zero-copy view; ``copy=True`` runs the library's flatten_forward instead."""

    def __init__(self, inputs, outputs, axis=1, dtype="float32", version="17", copy=False):
        super().__init__(inputs, outputs)
        self.axis, self.dtype, self.version, self.copy = axis, dtype, version, copy

    def _calc_shape(self, input_shape):
        axis = self.axis if self.axis >= 0 else len(input_shape) + self.axis
        lead = int(np.prod(input_shape[:axis], dtype=np.int64)) if axis > 0 else 1
        rest = int(np.prod(input_shape[axis:], dtype=np.int64)) if axis < len(input_shape) else 1
        return (lead, rest)

    def forward(self, input: Tensor) -> dict:
        out_shape = self._calc_shape(tuple(input.data.shape))
        if self.copy:
            x = self._numpy_to_ctensor(input.data, self.dtype)
            y = self._new_output(out_shape, self.dtype)
            self.lib.flatten_forward(x, y)
            return self._publish(self._finish([x], y, out_shape, self.dtype))
        dev = input.data if isinstance(input.data, DeviceArray) else DeviceArray.from_numpy(input.data, self.dtype, self.lib)
        out = dev.reshape(out_shape)
        capi.check(self.lib)
        return self._publish(Tensor(*out_shape, dtype=self.dtype, data=out))

    def forward_(self, input: Tensor_) -> dict:
        return self._publish(Tensor_(*self._calc_shape(input.size), dtype=self.dtype))


class Reshape(Flatten):
    """Reshape to an explicit shape (zero-copy); the library's reshape_forward is the same byte
    copy as flatten_forward (tensor_ops.c:1297-1299)."""

    def __init__(self, inputs, outputs, shape, dtype="float32", version="17"):
        super().__init__(inputs, outputs, axis=1, dtype=dtype, version=version)
        self.shape = tuple(shape)

    def _calc_shape(self, input_shape):
        total = int(np.prod(input_shape, dtype=np.int64))
        shape = list(self.shape)
        if -1 in shape:
            known = int(np.prod([s for s in shape if s != -1], dtype=np.int64))
            shape[shape.index(-1)] = total // known if known else 0
        return tuple(int(s) for s in shape)


# ---- operators around the hot path in exported CNNs ------------------------------------------------------------
class Cast(_Unary):
    """Element-wise conversion to ``dtype`` (nn/Operators.py:1270-1280)."""
    _c_name = "cast_forward"


class Clip(Ops):
    """min(max(x, min), max) with optional bounds that broadcast against x (nn/Operators.py:1282-1340)."""

    def __init__(self, inputs, outputs, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype
        self.version = version

    def forward(self, input: Tensor, min_val: Tensor = None, max_val: Tensor = None) -> dict:
        shapes = [self._shape_of(t) for t in (input, min_val, max_val) if t is not None]
        out_shape = np.broadcast_shapes(*shapes)
        out_dtype = self.dtype if self.dtype else input.dtype
        operands = [t for t in (input, min_val, max_val) if t is not None]
        handles = {id(t): self._numpy_to_ctensor(t.data, t.dtype) for t in operands}
        y = self._new_output(out_shape, out_dtype)
        self.lib.clip_forward(handles[id(input)], y, handles[id(min_val)] if min_val is not None else None,
                              handles[id(max_val)] if max_val is not None else None)
        return self._publish(self._finish(list(handles.values()), y, out_shape, out_dtype))

    def forward_(self, input: Tensor_, min_val: Tensor_ = None, max_val: Tensor_ = None) -> dict:
        return self._publish(Tensor_(*input.size, dtype=self.dtype))


class AveragePool(MaxPool):
    """Average pooling over NCHW (nn/Operators.py:2895-2960)."""

    def __init__(self, inputs, outputs, kernel_shape, pads, strides, dtype, dilations=[1, 1], count_include_pad=0, version="17"):
        super().__init__(inputs, outputs, kernel_shape, pads, strides, dtype, dilations, version)
        self.count_include_pad = count_include_pad

    def forward(self, x: Tensor) -> dict:
        n, c, h, w = x.data.shape
        out_shape = (n, c,
                     _pooled_extent(h, self.pads[0], self.pads[2], self.dilations[0], self.kernel_shape[0], self.strides[0]),
                     _pooled_extent(w, self.pads[1], self.pads[3], self.dilations[1], self.kernel_shape[1], self.strides[1]))
        keep = [_int_ptr(self.pads), _int_ptr(self.strides), _int_ptr(self.dilations), _int_ptr(self.kernel_shape)]
        params = CPoolParams(keep[0][1], keep[1][1], keep[2][1], keep[3][1])
        xh = self._numpy_to_ctensor(x.data, x.dtype)
        y = self._new_output(out_shape, self.dtype)
        self.lib.average_pool_forward(xh, y, ctypes.byref(params), int(self.count_include_pad))
        return self._publish(self._finish([xh], y, out_shape, self.dtype))


class GlobalAveragePool(Ops):
    """Mean over H x W of a 4-D tensor, output [N, C, 1, 1] (nn/Operators.py:2998-3025)."""

    def __init__(self, inputs, outputs, dtype="float32", version="17"):
        super().__init__(inputs, outputs)
        self.dtype = dtype
        self.version = version

    def forward(self, x: Tensor) -> dict:
        n, c = x.data.shape[:2]
        out_shape = (n, c, 1, 1)
        xh = self._numpy_to_ctensor(x.data, x.dtype)
        y = self._new_output(out_shape, self.dtype)
        self.lib.global_average_pool_forward(xh, y)
        return self._publish(self._finish([xh], y, out_shape, self.dtype))

    def forward_(self, x: Tensor_) -> dict:
        return self._publish(Tensor_(x.size[0], x.size[1], 1, 1, dtype=self.dtype))


class BatchNormalization(Ops):
    """Inference batch normalisation over dimension 1 (nn/Operators.py:3281-3320)."""

    def __init__(self, inputs, outputs, epsilon=1e-5, momentum=0.9, dtype="float32", version="17"):
        super().__init__(inputs, outputs)
        self.epsilon, self.momentum, self.dtype, self.version = epsilon, momentum, dtype, version

    def forward(self, x: Tensor, scale: Tensor, B: Tensor, mean: Tensor, var: Tensor) -> dict:
        shape = self._shape_of(x)
        handles = [self._numpy_to_ctensor(t.data, t.dtype) for t in (x, scale, B, mean, var)]
        y = self._new_output(shape, self.dtype)
        self.lib.batch_norm_forward(handles[0], handles[1], handles[2], handles[3], handles[4], y, ctypes.c_float(self.epsilon))
        return self._publish(self._finish(handles, y, shape, self.dtype))

    def forward_(self, x: Tensor_, *_) -> dict:
        return self._publish(Tensor_(*x.size, dtype=self.dtype))


# ---- element-wise families beyond the hot path (same templates, more expressions) -------------------------------------
class Max(_Binary):
    """Element-wise maximum with broadcasting (nn/Operators.py:933-949)."""
    _c_name = "max_forward"


class Min(_Binary):
    """Element-wise minimum with broadcasting (nn/Operators.py:951-967)."""
    _c_name = "min_forward"


class Pow(_Binary):
    """a ** b in double with broadcasting (nn/Operators.py:914-931)."""
    _c_name = "pow_forward"


def _unary_class(name, c_name, where):
    return type(name, (_Unary,), {"_c_name": c_name, "__doc__": f"Element-wise {c_name[:-8]} ({where})."})


EXP = _unary_class("EXP", "exp_forward", "nn/Operators.py:706-718")
LOG = _unary_class("LOG", "log_forward", "nn/Operators.py:720-732")
SQRT = _unary_class("SQRT", "sqrt_forward", "nn/Operators.py:734-746")
SIGMOID = _unary_class("SIGMOID", "sigmoid_forward", "nn/Operators.py:748-760")
TANH = _unary_class("TANH", "tanh_forward", "nn/Operators.py:762-774")
Neg = _unary_class("Neg", "neg_forward", "nn/Operators.py:1222-1232")
Reciprocal = _unary_class("Reciprocal", "reciprocal_forward", "nn/Operators.py:1234-1244")
Ceil = _unary_class("Ceil", "ceil_forward", "nn/Operators.py:1246-1256")
Floor = _unary_class("Floor", "floor_forward", "nn/Operators.py:1258-1268")
Sin = _unary_class("Sin", "sin_forward", "nn/Operators.py:1733-1741")
Tan = _unary_class("Tan", "tan_forward", "nn/Operators.py:1743-1751")
Atan = _unary_class("Atan", "atan_forward", "nn/Operators.py:1753-1761")
Softplus = _unary_class("Softplus", "softplus_forward", "nn/Operators.py:2709-2715")
Softsign = _unary_class("Softsign", "softsign_forward", "nn/Operators.py:2717-2723")
HardSwish = _unary_class("HardSwish", "hard_swish_forward", "nn/Operators.py:2725-2731")
Acos = _unary_class("Acos", "acos_forward", "nn/Operators.py:2733-2739")
Asin = _unary_class("Asin", "asin_forward", "nn/Operators.py:2741-2747")
Cosh = _unary_class("Cosh", "cosh_forward", "nn/Operators.py:2749-2755")
Sinh = _unary_class("Sinh", "sinh_forward", "nn/Operators.py:2757-2763")
Asinh = _unary_class("Asinh", "asinh_forward", "nn/Operators.py:2765-2771")
Acosh = _unary_class("Acosh", "acosh_forward", "nn/Operators.py:2773-2779")
Atanh = _unary_class("Atanh", "atanh_forward", "nn/Operators.py:2781-2787")
Round = _unary_class("Round", "round_forward", "nn/Operators.py:3265-3271")
Erf = _unary_class("Erf", "erf_forward", "nn/Operators.py:3273-3279")
Gelu = _unary_class("Gelu", "gelu_forward", "nn/Operators.py:3582-3596")


# ---- MatMul and DynamicQuantizeLinear ----------------------------------------------------------------------------------
def _matmul_shapes(shape_a, shape_b):
    """(library shapes of A and B, library output shape, final shape) with numpy's rules for 1-D operands
    (nn/Operators.py:1367-1425)."""
    a_1d, b_1d = len(shape_a) == 1, len(shape_b) == 1
    sa = [1] + list(shape_a) if a_1d else list(shape_a)
    sb = list(shape_b) + [1] if b_1d else list(shape_b)
    if sa[-1] != sb[-2]:
        raise ValueError(f"MatMul shape mismatch: {sa[-1]} != {sb[-2]} (Original shapes: A={tuple(shape_a)}, B={tuple(shape_b)})")
    try:
        batch = np.broadcast_shapes(tuple(sa[:-2]), tuple(sb[:-2]))
    except ValueError:
        raise ValueError(f"MatMul batch broadcast failed: {sa[:-2]} vs {sb[:-2]}")
    out = list(batch) + [sa[-2], sb[-1]]
    final = list(out)
    if b_1d:
        final.pop(-1)
    if a_1d:
        final.pop(-1 if b_1d else -2)
    return tuple(sa), tuple(sb), tuple(out), tuple(final)


class MatMul(Ops):
    """numpy-style matrix product: 1-D operands are promoted, leading dimensions broadcast (nn/Operators.py:1361-1432)."""

    def __init__(self, inputs, outputs, dtype, version="17"):
        super().__init__(inputs, outputs)
        self.dtype, self.version = dtype, version

    def forward(self, input_a: Tensor, input_b: Tensor) -> dict:
        sa, sb, out_shape, final = _matmul_shapes(self._shape_of(input_a), self._shape_of(input_b))
        data_a = input_a.data if tuple(input_a.data.shape) == sa else input_a.data.reshape(*sa)
        data_b = input_b.data if tuple(input_b.data.shape) == sb else input_b.data.reshape(*sb)
        handles = [self._numpy_to_ctensor(data_a, input_a.dtype), self._numpy_to_ctensor(data_b, input_b.dtype)]
        y = self._new_output(out_shape, self.dtype)
        self.lib.matmul_forward(handles[0], handles[1], y)
        result = self._finish(handles, y, out_shape, self.dtype)
        if final != out_shape:
            result = Tensor(*final, dtype=self.dtype, data=result.data.reshape(*final))
        return self._publish(result)

    def forward_(self, input_a: Tensor_, input_b: Tensor_) -> dict:
        return self._publish(Tensor_(*_matmul_shapes(tuple(input_a.size), tuple(input_b.size))[3], dtype=self.dtype))


class DynamicQuantizeLinear(Ops):
    """uint8 codes with the scale and zero point taken from the tensor's own range (nn/Operators.py:3892-3925).
    Returns [y, y_scale, y_zero_point]."""

    def __init__(self, inputs, outputs, dtype="uint8", version="17"):
        super().__init__(inputs, outputs)
        self.dtype, self.version = "uint8", version

    def forward(self, x: Tensor) -> dict:
        shape = self._shape_of(x)
        xh = self._numpy_to_ctensor(x.data, x.dtype)
        outs = [self._new_output(shape, "uint8"), self._new_output((1,), "float32"), self._new_output((1,), "uint8")]
        self.lib.dynamic_quantize_linear_forward(xh, outs[0], outs[1], outs[2])
        y = self._finish([xh], outs[0], shape, "uint8")
        scale = self._finish([], outs[1], (1,), "float32")
        zero = self._finish([], outs[2], (1,), "uint8")
        return self._publish([y, scale, zero])

    def forward_(self, x: Tensor_) -> dict:
        return self._publish([Tensor_(*x.size, dtype="uint8"), Tensor_(1, dtype="float32"), Tensor_(1, dtype="uint8")])
