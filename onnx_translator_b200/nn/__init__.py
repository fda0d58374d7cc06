"""Host-side operator interface, mirroring the reference's ``nn`` package for the hot path.

Same public names and meanings as the reference (nn/__init__.py:9-344): ``Tensor`` (real data),
``Tensor_`` (shape/dtype placeholder), ``Ops`` (base class that owns the C library handle and the
unary / binary / ternary execution templates), the dtype tables.  The difference is residency:
``Tensor.data`` may be a numpy array (uploaded when first used) or a ``DeviceArray``; every
operator returns a ``Tensor`` whose ``data`` is a ``DeviceArray``, so a chain of operators never
copies through the host.  ``numpy.asarray(t.data)`` downloads a result.

Broadcasting is not materialised: the library's binary and Q/DQ entry points take operands of
different shapes and index them with stride-0 dimensions.
"""
from __future__ import annotations

import ctypes
from typing import Optional

import numpy as np

from .. import capi
from ..capi import CTensor, DTYPE_MAP, DTYPE_TO_NUMPY, NUMPY_TO_DTYPE  # noqa: F401  (re-exported)
from ..device import DeviceArray


def _size_tuple(size):
    return tuple(size[0]) if (len(size) == 1 and isinstance(size[0], (list, tuple))) else tuple(size)


class Tensor:
    """Data-carrying tensor: ``size`` (shape tuple), ``data_size``, ``dtype`` (name), ``data``."""

    def __init__(self, *size, dtype="float32", data=None):
        self.size = _size_tuple(size)
        self.data_size = int(np.prod(self.size, dtype=np.int64)) if len(self.size) else 1
        self.dtype = dtype
        self.data = data if data is not None else np.zeros(self.size, dtype=DTYPE_TO_NUMPY[dtype])

    def numpy(self) -> np.ndarray:
        """Host copy of the contents in the storage convention of ``dtype``."""
        return self.data.numpy() if isinstance(self.data, DeviceArray) else np.asarray(self.data)

    def to_device(self) -> "Tensor":
        if not isinstance(self.data, DeviceArray):
            self.data = DeviceArray.from_numpy(self.data, self.dtype)
        return self


class Tensor_:
    """Placeholder used by the shape-only pass (``forward_``)."""

    def __init__(self, *size, dtype="float32"):
        self.size = _size_tuple(size)
        self.data_size = int(np.prod(self.size, dtype=np.int64)) if len(self.size) else 1
        self.dtype = dtype


class Ops:
    """Base of every operator class; holds the library and the execution templates."""
    _lib = None
    _recorder = None                         # set while a call plan is being recorded (nn/plan.py)

    @classmethod
    def _get_lib(cls):
        if Ops._lib is None:
            lib = capi.load()                # raises when the CUDA library is not built
            lib.init_cos_lut()
            capi.check(lib)                  # raises when there is no usable CUDA device
            Ops._lib = lib
        return Ops._lib

    def __init__(self, inputs, outputs):
        self.inputs = inputs
        self.outputs = outputs
        self.parameters = {}
        self.name = None
        self.dtype = None

    @property
    def lib(self):
        """The operator library, opened at the first use: a node can be constructed (and a graph built and
        inspected) on a machine without a GPU; running it there raises."""
        return Ops._recorder or self._get_lib()

    # -- marshalling ---------------------------------------------------------------------------
    def _numpy_to_ctensor(self, arr, dtype: str):
        """Tensor handle for an operand.  A DeviceArray is borrowed (one more reference, no
        copy); a host array is uploaded.  Either way the caller releases it with free_tensor."""
        if isinstance(arr, DeviceArray):
            self.lib.tops_retain(arr.handle)
            return arr.handle
        dev = DeviceArray.from_numpy(np.asarray(arr), dtype, self.lib)
        handle, dev.handle = dev.handle, None        # hand the only reference to the caller
        return handle

    def _ctensor_to_numpy(self, c_tensor, dtype: str) -> DeviceArray:
        """Adopt an output tensor without copying; the caller's free_tensor drops its own
        reference and the returned DeviceArray keeps the memory alive."""
        self.lib.tops_retain(c_tensor)
        return DeviceArray(c_tensor, dtype, self.lib)

    def _new_output(self, shape, dtype: str):
        arr, nd = capi.shape_array(shape)
        handle = self.lib.tops_create_uninit(arr, nd, DTYPE_MAP[dtype])
        if not handle:
            capi.check(self.lib)
            raise capi.TensorOpsError("output allocation failed")
        return handle

    @staticmethod
    def _shape_of(t) -> tuple:
        return tuple(t.data.shape)

    def _finish(self, handles, out_handle, out_shape, out_dtype) -> Tensor:
        out = self._ctensor_to_numpy(out_handle, out_dtype)
        for h in handles:
            self.lib.free_tensor(h)
        self.lib.free_tensor(out_handle)
        capi.check(self.lib)
        return Tensor(*out_shape, dtype=out_dtype, data=out)

    # -- execution templates (nn/__init__.py:189-279) ---------------------------------------------------
    def _execute_unary(self, input_tensor, c_func_name):
        out_dtype = self.dtype if self.dtype else input_tensor.dtype
        shape = self._shape_of(input_tensor)
        x = self._numpy_to_ctensor(input_tensor.data, input_tensor.dtype)
        y = self._new_output(shape, out_dtype)
        getattr(self.lib, c_func_name)(x, y)
        return self._finish([x], y, shape, out_dtype)

    def _execute_binary(self, input_a, input_b, c_func_name):
        try:
            out_shape = np.broadcast_shapes(self._shape_of(input_a), self._shape_of(input_b))
        except ValueError:
            print(f"Broadcasting error: {input_a.size} vs {input_b.size}")
            raise
        if self.dtype:
            out_dtype = self.dtype
        else:       # promotion over the STORAGE types, as the reference does
            res = np.result_type(DTYPE_TO_NUMPY[input_a.dtype], DTYPE_TO_NUMPY[input_b.dtype])
            out_dtype = NUMPY_TO_DTYPE.get(res.type, "float32")
        a = self._numpy_to_ctensor(input_a.data, input_a.dtype)
        b = self._numpy_to_ctensor(input_b.data, input_b.dtype)
        o = self._new_output(out_shape, out_dtype)
        getattr(self.lib, c_func_name)(a, b, o)
        return self._finish([a, b], o, out_shape, out_dtype)

    def _execute_ternary(self, in_a, in_b, in_c, c_func_name):
        try:
            out_shape = np.broadcast_shapes(self._shape_of(in_a), self._shape_of(in_b), self._shape_of(in_c))
        except ValueError:
            print(f"Broadcasting error in ternary op: {in_a.size}, {in_b.size}, {in_c.size}")
            raise
        out_dtype = self.dtype if self.dtype else "float32"
        a = self._numpy_to_ctensor(in_a.data, in_a.dtype)
        b = self._numpy_to_ctensor(in_b.data, in_b.dtype)
        c = self._numpy_to_ctensor(in_c.data, in_c.dtype)
        o = self._new_output(out_shape, out_dtype)
        getattr(self.lib, c_func_name)(a, b, c, o)
        return self._finish([a, b, c], o, out_shape, out_dtype)

    def _publish(self, out_tensor):
        values = {"tensor": out_tensor, "parameters": None, "graph": None}
        self.parameters = {"values": values}
        return values

    def forward(self, input):
        pass

    def forward_(self, input):
        pass


def synchronize() -> None:
    """Wait for every operator enqueued so far on the current device."""
    lib = Ops._get_lib()
    lib.tops_sync()
    capi.check(lib)


from .graph import Graph, qdq_resnet50, small_cnn  # noqa: E402  (the graph runner builds on the classes above)
from .plan import GraphPlan  # noqa: E402
