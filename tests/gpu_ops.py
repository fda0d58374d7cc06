"""Runs operators on the GPU through the package's operator classes (which call the C ABI) and
returns host arrays, with the same call shapes as ``oracle.HostOracle`` so a parity test is
``assert_same_codes(gpu.op(...), port.op(...))``."""
from __future__ import annotations

import numpy as np

from onnx_translator_b200 import nn
from onnx_translator_b200.nn import Operators as ops

_UNARY = {"relu": ops.RELU, "abs": ops.ABS, "cos": ops.COS}
_BINARY = {"add": ops.ADD, "sub": ops.SUB, "mul": ops.MUL, "div": ops.DIV}


def _t(arr, dt):
    arr = np.asarray(arr)
    return nn.Tensor(*arr.shape, dtype=dt, data=arr)


def unary(op, x, x_dt, out_dt):
    return _UNARY[op]([], [], dtype=out_dt).forward(_t(x, x_dt))["tensor"].numpy()


def binary(op, a, a_dt, b, b_dt, out_dt):
    return _BINARY[op]([], [], dtype=out_dt).forward(_t(a, a_dt), _t(b, b_dt))["tensor"].numpy()


def quantize(x, x_dt, s, s_dt, z, z_dt, out_dt, axis=None):
    node = ops.QuantizeLinear([], [], axis=1 if axis is None else axis, dtype=out_dt)
    return node.forward(_t(x, x_dt), _t(s, s_dt), _t(z, z_dt))["tensor"].numpy()


def dequantize(x, x_dt, s, s_dt, z, z_dt, out_dt):
    return ops.DequantizeLinear([], [], dtype=out_dt).forward(_t(x, x_dt), _t(s, s_dt), _t(z, z_dt))["tensor"].numpy()


def conv2d(x, x_dt, w, w_dt, b, b_dt, out_dt, pads, strides, dilations, group):
    node = ops.Conv([], [], pads=list(pads), strides=list(strides), dilations=list(dilations), group=group, dtype=out_dt)
    bias = None if b is None else _t(b, b_dt)
    return node.forward(_t(x, x_dt), _t(w, w_dt), bias)["tensor"].numpy()


def max_pool(x, x_dt, out_dt, kernel, pads, strides, dilations=(1, 1)):
    node = ops.MaxPool([], [], kernel_shape=list(kernel), pads=list(pads), strides=list(strides), dtype=out_dt,
                       dilations=list(dilations))
    return node.forward(_t(x, x_dt))["tensor"].numpy()


def gemm(a, a_dt, b, b_dt, c, c_dt, out_dt, alpha=1.0, beta=1.0, transA=0, transB=0):
    node = ops.Gemm([], [], alpha=alpha, beta=beta, transA=transA, transB=transB, dtype=out_dt)
    cc = None if c is None else _t(c, c_dt)
    return node.forward(_t(a, a_dt), _t(b, b_dt), cc)["tensor"].numpy()


def softmax(x, x_dt, out_dt, axis=-1):
    return ops.Softmax([], [], axis=axis, dtype=out_dt).forward(_t(x, x_dt))["tensor"].numpy()


def flatten(x, x_dt, out_shape, copy=True):
    node = ops.Flatten([], [], axis=1, dtype=x_dt, copy=copy)
    out = node.forward(_t(x, x_dt))["tensor"].numpy()
    return out.reshape(out_shape)


# ---- operators around the hot path -------------------------------------------------------------------------------
def cast(x, x_dt, out_dt):
    return ops.Cast([], [], dtype=out_dt).forward(_t(x, x_dt))["tensor"].numpy()


def clip(x, x_dt, lo, lo_dt, hi, hi_dt, out_dt):
    lo_t = None if lo is None else _t(lo, lo_dt)
    hi_t = None if hi is None else _t(hi, hi_dt)
    return ops.Clip([], [], dtype=out_dt).forward(_t(x, x_dt), lo_t, hi_t)["tensor"].numpy()


def average_pool(x, x_dt, out_dt, kernel, pads, strides, dilations=(1, 1), count_include_pad=0):
    node = ops.AveragePool([], [], kernel_shape=list(kernel), pads=list(pads), strides=list(strides), dtype=out_dt,
                           dilations=list(dilations), count_include_pad=count_include_pad)
    return node.forward(_t(x, x_dt))["tensor"].numpy()


def global_average_pool(x, x_dt, out_dt):
    return ops.GlobalAveragePool([], [], dtype=out_dt).forward(_t(x, x_dt))["tensor"].numpy()


def batch_norm(x, x_dt, scale, bias, mean, var, p_dt, out_dt, epsilon=1e-5):
    node = ops.BatchNormalization([], [], epsilon=epsilon, dtype=out_dt)
    return node.forward(_t(x, x_dt), _t(scale, p_dt), _t(bias, p_dt), _t(mean, p_dt), _t(var, p_dt))["tensor"].numpy()


_BINARY.update({"max": ops.Max, "min": ops.Min, "pow": ops.Pow})
_MATH = {"exp": ops.EXP, "log": ops.LOG, "sqrt": ops.SQRT, "sigmoid": ops.SIGMOID, "tanh": ops.TANH, "neg": ops.Neg,
         "reciprocal": ops.Reciprocal, "ceil": ops.Ceil, "floor": ops.Floor, "sin": ops.Sin, "tan": ops.Tan, "atan": ops.Atan,
         "softplus": ops.Softplus, "softsign": ops.Softsign, "hard_swish": ops.HardSwish, "acos": ops.Acos, "asin": ops.Asin,
         "cosh": ops.Cosh, "sinh": ops.Sinh, "asinh": ops.Asinh, "acosh": ops.Acosh, "atanh": ops.Atanh, "round": ops.Round,
         "erf": ops.Erf, "gelu": ops.Gelu}


def unary_math(op, x, x_dt, out_dt):
    return _MATH[op]([], [], dtype=out_dt).forward(_t(x, x_dt))["tensor"].numpy()


def matmul(a, a_dt, b, b_dt, out_dt):
    return ops.MatMul([], [], dtype=out_dt).forward(_t(a, a_dt), _t(b, b_dt))["tensor"].numpy()


def dynamic_quantize_linear(x, x_dt):
    y, scale, zero = ops.DynamicQuantizeLinear([], []).forward(_t(x, x_dt))["tensor"]
    return y.numpy(), scale.numpy(), zero.numpy()
