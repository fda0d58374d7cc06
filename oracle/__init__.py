"""Host-side checker libraries for the parity tests.  TEST INFRASTRUCTURE ONLY.

Two shared objects can be driven through the same small numpy API:

* ``HostOracle("port")`` -- ``oracle/_build/liboracle.so``, the independent C restatement in
  ``oracle/oracle.c`` (always buildable: one C file, gcc + OpenMP).
* ``HostOracle("ref")``  -- ``oracle/_ref/tensor_ops_ref.so``, the reference project's own
  ``tensor_ops/tensor_ops.c`` compiled unchanged by ``oracle/Makefile`` (present only where the
  reference sources were available at build time, or where the prebuilt file travelled along).

Only tests, the smoke check and the CPU-baseline leg of the benchmark may import this package;
the product never does.  Arrays use the reference's storage convention
(nn/__init__.py:37-51): fp8 codes as uint8, bfloat16 codes as uint16, int4 one value per int8.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from typing import Optional, Sequence

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
PORT_SO = os.path.join(HERE, "_build", "liboracle.so")
REF_SO = os.path.join(HERE, "_ref", "tensor_ops_ref.so")

# tensor_ops/tensor_ops.h:10-23 and nn/__init__.py:20-51
DTYPE_CODE = {
    "float8_e4m3": 0, "float8_e5m2": 1, "float16": 2, "bfloat16": 3, "float32": 4, "float64": 5,
    "int4": 6, "int8": 7, "uint8": 8, "int16": 9, "int32": 10, "int64": 11,
}
DTYPE_STORAGE = {
    "float8_e4m3": np.uint8, "float8_e5m2": np.uint8, "float16": np.float16, "bfloat16": np.uint16,
    "float32": np.float32, "float64": np.float64, "int4": np.int8, "int8": np.int8,
    "uint8": np.uint8, "int16": np.int16, "int32": np.int32, "int64": np.int64,
}


class _CTensor(ctypes.Structure):
    _fields_ = [("data", ctypes.c_void_p), ("shape", ctypes.POINTER(ctypes.c_int)),
                ("ndim", ctypes.c_int), ("size", ctypes.c_size_t), ("dtype", ctypes.c_int)]


class _CConvParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("group", ctypes.c_int)]


class _CPoolParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("kernel_shape", ctypes.POINTER(ctypes.c_int))]


def build(quiet: bool = True) -> None:
    """Run ``make -C oracle`` (the port always; the reference build when its sources exist)."""
    subprocess.run(["make", "-C", HERE], check=True,
                   stdout=subprocess.DEVNULL if quiet else None)


def available(kind: str) -> bool:
    return os.path.exists(PORT_SO if kind == "port" else REF_SO)


def use_all_host_threads() -> int:
    """Sets the OpenMP team of the libraries loaded from here to every core this process may run on
    (a launcher may have exported OMP_NUM_THREADS=1) and returns that count."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    try:
        ctypes.CDLL("libgomp.so.1").omp_set_num_threads(ctypes.c_int(n))
    except OSError:
        return int(os.environ.get("OMP_NUM_THREADS", "1"))
    return n


def _ints(values: Sequence[int]):
    return (ctypes.c_int * len(values))(*[int(v) for v in values])


class _Wrapped:
    """A numpy array viewed as the C ``Tensor`` struct (borrowing the array's memory)."""

    def __init__(self, arr: np.ndarray, dtype: str):
        storage = DTYPE_STORAGE[dtype]
        self.arr = np.ascontiguousarray(arr, dtype=storage)
        self.shape = _ints(self.arr.shape if self.arr.ndim else ())
        self.c = _CTensor(self.arr.ctypes.data, ctypes.cast(self.shape, ctypes.POINTER(ctypes.c_int)),
                          self.arr.ndim, self.arr.size, DTYPE_CODE[dtype])

    @property
    def ref(self):
        return ctypes.byref(self.c)


def _out(shape, dtype: str) -> _Wrapped:
    return _Wrapped(np.zeros(shape, dtype=DTYPE_STORAGE[dtype]), dtype)


class HostOracle:
    """Uniform numpy front for either checker library."""

    _NAMES = {
        "port": dict(relu="orc_relu", abs="orc_abs", cos="orc_cos", add="orc_add", sub="orc_sub",
                     mul="orc_mul", div="orc_div", quantize="orc_quantize_linear",
                     dequantize="orc_dequantize_linear", conv="orc_conv2d", pool="orc_max_pool",
                     gemm="orc_gemm", softmax="orc_softmax", flatten="orc_flatten",
                     cast="orc_cast", clip="orc_clip", average_pool="orc_average_pool",
                     global_average_pool="orc_global_average_pool", batch_norm="orc_batch_norm",
                     max="orc_max", min="orc_min", pow="orc_pow", matmul="orc_matmul",
                     dynamic_quantize="orc_dynamic_quantize_linear", init="orc_init_cos_lut"),
        "ref": dict(relu="relu_forward", abs="abs_forward", cos="cos_forward", add="add_forward",
                    sub="sub_forward", mul="mul_forward", div="div_forward",
                    quantize="quantize_linear_forward", dequantize="dequantize_linear_forward",
                    conv="conv2d_forward", pool="max_pool_forward", gemm="gemm_forward",
                    softmax="softmax_forward", flatten="flatten_forward", cast="cast_forward", clip="clip_forward",
                    average_pool="average_pool_forward", global_average_pool="global_average_pool_forward",
                    batch_norm="batch_norm_forward", max="max_forward", min="min_forward", pow="pow_forward",
                    matmul="matmul_forward", dynamic_quantize="dynamic_quantize_linear_forward",
                    init="init_cos_lut"),
    }

    def __init__(self, kind: str = "port"):
        if kind not in self._NAMES:
            raise ValueError(kind)
        path = PORT_SO if kind == "port" else REF_SO
        if not os.path.exists(path):
            build()
        if not os.path.exists(path):
            raise FileNotFoundError(path)
        self.kind = kind
        self.lib = ctypes.CDLL(path)
        self._fn = {k: getattr(self.lib, v) for k, v in self._NAMES[kind].items()}
        for f in self._fn.values():
            f.restype = None
        self._fn["gemm"].argtypes = [ctypes.c_void_p] * 4 + [ctypes.c_float, ctypes.c_float,
                                                             ctypes.c_int, ctypes.c_int]
        self._fn["softmax"].argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        self._fn["average_pool"].argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int]
        self._fn["batch_norm"].argtypes = [ctypes.c_void_p] * 6 + [ctypes.c_float]
        self._fn["init"]()
        if kind == "port":
            self.lib.orc_encode.restype = ctypes.c_uint32
            self.lib.orc_encode.argtypes = [ctypes.c_int, ctypes.c_float]
            self.lib.orc_decode.restype = ctypes.c_float
            self.lib.orc_decode.argtypes = [ctypes.c_int, ctypes.c_uint32]
            self.lib.orc_cos_table.restype = ctypes.POINTER(ctypes.c_double)

    # -- elementwise ---------------------------------------------------------------------
    def unary(self, op: str, x, x_dt: str, out_dt: str) -> np.ndarray:
        xi = _Wrapped(x, x_dt)
        yo = _out(xi.arr.shape, out_dt)
        self._fn[op](xi.ref, yo.ref)
        return yo.arr

    def binary(self, op: str, a, a_dt: str, b, b_dt: str, out_dt: str) -> np.ndarray:
        """Operands are broadcast on the host first, as nn/__init__.py:210-248 does."""
        a = np.asarray(a, dtype=DTYPE_STORAGE[a_dt])
        b = np.asarray(b, dtype=DTYPE_STORAGE[b_dt])
        ab, bb = np.broadcast_arrays(a, b)
        ai, bi = _Wrapped(ab, a_dt), _Wrapped(bb, b_dt)
        yo = _out(ab.shape, out_dt)
        self._fn[op](ai.ref, bi.ref, yo.ref)
        return yo.arr

    def _ternary(self, op, x, x_dt, s, s_dt, z, z_dt, out_dt):
        x = np.asarray(x, dtype=DTYPE_STORAGE[x_dt])
        s = np.asarray(s, dtype=DTYPE_STORAGE[s_dt])
        z = np.asarray(z, dtype=DTYPE_STORAGE[z_dt])
        xb, sb, zb = np.broadcast_arrays(x, s, z)
        xi, si, zi = _Wrapped(xb, x_dt), _Wrapped(sb, s_dt), _Wrapped(zb, z_dt)
        yo = _out(xb.shape, out_dt)
        self._fn[op](xi.ref, si.ref, zi.ref, yo.ref)
        return yo.arr

    def quantize(self, x, x_dt, s, s_dt, z, z_dt, out_dt, axis: Optional[int] = None):
        """``axis`` reshapes 1-D scale/zero-point like nn/Operators.py:439-445."""
        x = np.asarray(x)
        s, z = np.asarray(s), np.asarray(z)
        if axis is not None and s.ndim == 1 and x.ndim > 1:
            shape = [1] * x.ndim
            shape[axis if axis >= 0 else axis + x.ndim] = s.size
            s, z = s.reshape(shape), z.reshape(shape)
        return self._ternary("quantize", x, x_dt, s, s_dt, z, z_dt, out_dt)

    def dequantize(self, x, x_dt, s, s_dt, z, z_dt, out_dt):
        return self._ternary("dequantize", x, x_dt, s, s_dt, z, z_dt, out_dt)

    # -- structured ops --------------------------------------------------------------------
    def conv2d(self, x, x_dt, w, w_dt, b, b_dt, out_dt, pads, strides, dilations, group):
        xi, wi = _Wrapped(x, x_dt), _Wrapped(w, w_dt)
        bi = _Wrapped(b, b_dt) if b is not None else None
        n, _, h, wd = xi.arr.shape
        m, _, kh, kw = wi.arr.shape
        oh = (h + pads[0] + pads[2] - dilations[0] * (kh - 1) - 1) // strides[0] + 1
        ow = (wd + pads[1] + pads[3] - dilations[1] * (kw - 1) - 1) // strides[1] + 1
        yo = _out((n, m, oh, ow), out_dt)
        keep = (_ints(pads), _ints(strides), _ints(dilations))
        prm = _CConvParams(ctypes.cast(keep[0], ctypes.POINTER(ctypes.c_int)),
                           ctypes.cast(keep[1], ctypes.POINTER(ctypes.c_int)),
                           ctypes.cast(keep[2], ctypes.POINTER(ctypes.c_int)), int(group))
        self._fn["conv"](xi.ref, wi.ref, bi.ref if bi is not None else None, yo.ref, ctypes.byref(prm))
        return yo.arr

    def max_pool(self, x, x_dt, out_dt, kernel, pads, strides, dilations=(1, 1)):
        xi = _Wrapped(x, x_dt)
        n, c, h, wd = xi.arr.shape
        oh = (h + pads[0] + pads[2] - dilations[0] * (kernel[0] - 1) - 1) // strides[0] + 1
        ow = (wd + pads[1] + pads[3] - dilations[1] * (kernel[1] - 1) - 1) // strides[1] + 1
        yo = _out((n, c, oh, ow), out_dt)
        keep = (_ints(pads), _ints(strides), _ints(dilations), _ints(kernel))
        prm = _CPoolParams(*[ctypes.cast(k, ctypes.POINTER(ctypes.c_int)) for k in keep])
        self._fn["pool"](xi.ref, yo.ref, ctypes.byref(prm))
        return yo.arr

    # The one-line unary operators: the port has one entry point with a selector, the reference one
    # function per operator.
    UNARY_MATH = ("exp", "log", "sqrt", "sigmoid", "tanh", "neg", "reciprocal", "ceil", "floor", "sin", "tan", "atan",
                  "softplus", "softsign", "hard_swish", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "round",
                  "erf", "gelu")

    def unary_math(self, op: str, x, x_dt: str, out_dt: str) -> np.ndarray:
        xi = _Wrapped(x, x_dt)
        yo = _out(xi.arr.shape, out_dt)
        if self.kind == "port":
            fn = self.lib.orc_unary_math
            fn.restype = None
            fn(ctypes.c_int(self.UNARY_MATH.index(op)), xi.ref, yo.ref)
        else:
            fn = getattr(self.lib, op + "_forward")
            fn.restype = None
            fn(xi.ref, yo.ref)
        return yo.arr

    # -- operators around the hot path ----------------------------------------------------------
    def cast(self, x, x_dt: str, out_dt: str) -> np.ndarray:
        return self.unary("cast", x, x_dt, out_dt)

    def clip(self, x, x_dt, lo, lo_dt, hi, hi_dt, out_dt) -> np.ndarray:
        """Bounds (either may be None) are broadcast to the input's shape first, as nn/Operators.py does."""
        xi = _Wrapped(x, x_dt)
        bounds = []
        for b, dt in ((lo, lo_dt), (hi, hi_dt)):
            bounds.append(None if b is None else _Wrapped(np.broadcast_to(np.asarray(b, dtype=DTYPE_STORAGE[dt]), xi.arr.shape), dt))
        yo = _out(xi.arr.shape, out_dt)
        self._fn["clip"](xi.ref, yo.ref, bounds[0].ref if bounds[0] else None, bounds[1].ref if bounds[1] else None)
        return yo.arr

    def average_pool(self, x, x_dt, out_dt, kernel, pads, strides, dilations=(1, 1), count_include_pad=0):
        xi = _Wrapped(x, x_dt)
        n, c, h, wd = xi.arr.shape
        oh = (h + pads[0] + pads[2] - dilations[0] * (kernel[0] - 1) - 1) // strides[0] + 1
        ow = (wd + pads[1] + pads[3] - dilations[1] * (kernel[1] - 1) - 1) // strides[1] + 1
        yo = _out((n, c, oh, ow), out_dt)
        keep = (_ints(pads), _ints(strides), _ints(dilations), _ints(kernel))
        prm = _CPoolParams(*[ctypes.cast(k, ctypes.POINTER(ctypes.c_int)) for k in keep])
        self._fn["average_pool"](xi.ref, yo.ref, ctypes.byref(prm), int(count_include_pad))
        return yo.arr

    def global_average_pool(self, x, x_dt, out_dt):
        xi = _Wrapped(x, x_dt)
        yo = _out(xi.arr.shape[:2] + (1, 1), out_dt)
        self._fn["global_average_pool"](xi.ref, yo.ref)
        return yo.arr

    def batch_norm(self, x, x_dt, scale, bias, mean, var, p_dt, out_dt, epsilon=1e-5):
        xi = _Wrapped(x, x_dt)
        ps = [_Wrapped(t, p_dt) for t in (scale, bias, mean, var)]
        yo = _out(xi.arr.shape, out_dt)
        self._fn["batch_norm"](xi.ref, ps[0].ref, ps[1].ref, ps[2].ref, ps[3].ref, yo.ref, ctypes.c_float(epsilon))
        return yo.arr

    def gemm(self, a, a_dt, b, b_dt, c, c_dt, out_dt, alpha=1.0, beta=1.0, transA=0, transB=0):
        ai, bi = _Wrapped(a, a_dt), _Wrapped(b, b_dt)
        m = ai.arr.shape[1] if transA else ai.arr.shape[0]
        n = bi.arr.shape[0] if transB else bi.arr.shape[1]
        ci = None
        if c is not None:
            c = np.asarray(c)
            if c.ndim == 1:                      # nn/Operators.py:640-645
                if c.shape[0] == n:
                    c = c.reshape(1, -1)
                elif c.shape[0] == m:
                    c = c.reshape(-1, 1)
            ci = _Wrapped(c, c_dt)
        yo = _out((m, n), out_dt)
        self._fn["gemm"](ctypes.addressof(ai.c), ctypes.addressof(bi.c),
                         ctypes.addressof(ci.c) if ci is not None else None,
                         ctypes.addressof(yo.c), float(alpha), float(beta), int(transA), int(transB))
        return yo.arr

    def matmul(self, a, a_dt, b, b_dt, out_dt):
        """Operands of rank >= 2 (the caller promotes 1-D operands, nn/Operators.py:1367-1377)."""
        ai, bi = _Wrapped(a, a_dt), _Wrapped(b, b_dt)
        batch = np.broadcast_shapes(ai.arr.shape[:-2], bi.arr.shape[:-2])
        yo = _out(tuple(batch) + (ai.arr.shape[-2], bi.arr.shape[-1]), out_dt)
        self._fn["matmul"](ai.ref, bi.ref, yo.ref)
        return yo.arr

    def dynamic_quantize_linear(self, x, x_dt, y_dt="uint8", scale_dt="float32", zp_dt="uint8"):
        """Returns (codes, scale[1], zero point[1])."""
        xi = _Wrapped(x, x_dt)
        yo, so, zo = _out(xi.arr.shape, y_dt), _out((1,), scale_dt), _out((1,), zp_dt)
        self._fn["dynamic_quantize"](xi.ref, yo.ref, so.ref, zo.ref)
        return yo.arr, so.arr, zo.arr

    def dynamic_quantize_range(self, x, x_dt) -> np.ndarray:
        """[min, max] of the elements as float64 (the restatement only: the reference has no such entry point)."""
        xi = _Wrapped(x, x_dt)
        out = np.zeros(2, np.float64)
        fn = self.lib.orc_dynamic_quantize_range
        fn.restype, fn.argtypes = None, [ctypes.c_void_p, ctypes.c_void_p]
        fn(xi.ref, out.ctypes.data)
        return out

    def dynamic_quantize_apply(self, x, x_dt, value_range, y_dt="uint8", scale_dt="float32", zp_dt="uint8"):
        xi = _Wrapped(x, x_dt)
        rng = np.ascontiguousarray(value_range, dtype=np.float64)
        yo, so, zo = _out(xi.arr.shape, y_dt), _out((1,), scale_dt), _out((1,), zp_dt)
        fn = self.lib.orc_dynamic_quantize_apply
        fn.restype, fn.argtypes = None, [ctypes.c_void_p] * 5
        fn(xi.ref, rng.ctypes.data, yo.ref, so.ref, zo.ref)
        return yo.arr, so.arr, zo.arr

    def softmax(self, x, x_dt, out_dt, axis=-1):
        xi = _Wrapped(x, x_dt)
        yo = _out(xi.arr.shape, out_dt)
        self._fn["softmax"](ctypes.addressof(xi.c), ctypes.addressof(yo.c), int(axis))
        return yo.arr

    def flatten(self, x, x_dt, out_shape):
        xi = _Wrapped(x, x_dt)
        yo = _out(tuple(out_shape), x_dt)
        self._fn["flatten"](xi.ref, yo.ref)
        return yo.arr

    # -- codec tables (port only) ------------------------------------------------------------
    def encode(self, dt: str, value: float) -> int:
        return int(self.lib.orc_encode(DTYPE_CODE[dt], float(value)))

    def decode(self, dt: str, code: int) -> float:
        return float(self.lib.orc_decode(DTYPE_CODE[dt], int(code)))

    def cos_table(self) -> np.ndarray:
        ptr = self.lib.orc_cos_table()
        return np.ctypeslib.as_array(ptr, shape=(4097,)).copy()
