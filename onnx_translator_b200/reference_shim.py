"""Binds the REFERENCE project's own ``nn`` package (its ``Ops`` base class and operator classes,
nn/__init__.py:134-344 and nn/Operators.py) to this library with device-resident tensors.

Without this module the reference's Python works against the library unchanged when the library is
in managed-memory mode (``tops_set_memory_mode(1)``): its ``_numpy_to_ctensor`` memmoves into
``Tensor.data`` and its ``_ctensor_to_numpy`` reads the result back through the pointer
(nn/__init__.py:305-344), which managed memory allows.  ``install(nn)`` is the product mode: it
replaces exactly the marshalling helpers and the three execution templates of ``nn.Ops``, so that

* an operand that already lives on the device (``Tensor.data`` is a ``DeviceArray``) is borrowed,
  not copied; a numpy operand is uploaded once;
* an operator's result is adopted as a ``DeviceArray`` instead of being copied to numpy;
* binary and Q/DQ operators hand their operands to the library as they are -- it broadcasts with
  zero strides -- instead of materialising them with ``numpy.broadcast_arrays`` (nn/__init__.py:213).

The reference's operator classes themselves (``Conv.forward``, ``MaxPool.forward``, ``Gemm.forward``,
``Softmax.forward``, ``Flatten.forward``, the ``ADD`` ... ``DIV`` / ``RELU`` / ``ABS`` / ``COS`` /
``QuantizeLinear`` / ``DequantizeLinear`` classes) run unmodified on top.  ``numpy.asarray(t.data)``
downloads a result.

The reference sets ``argtypes`` on the shared library object with its OWN ctypes struct classes
(nn/Operators.py:488, 561, 623, 678), so it gets a library object of its own here; handles cross
between the two sets of struct classes by pointer casts.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import capi
from .device import DeviceArray


def install(ref_nn, lib_path: str = None):
    """Patch ``ref_nn`` (the imported reference package ``nn``) in place and return its library object."""
    path = lib_path or capi.LIB_PATH
    capi.load()                                       # fails loudly when the CUDA library is not built
    lib = ctypes.CDLL(path)                           # same loaded image, separate Python function objects
    ref_ptr = ctypes.POINTER(ref_nn.CTensor)
    lib.create_tensor.restype = ref_ptr
    lib.create_tensor.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int]
    lib.tops_create_uninit.restype = ref_ptr
    lib.tops_create_uninit.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int]
    lib.free_tensor.argtypes = [ctypes.c_void_p]
    lib.tops_retain.argtypes = [ctypes.c_void_p]
    lib.tops_last_error.restype = ctypes.c_int
    lib.tops_last_error_message.restype = ctypes.c_char_p
    lib.init_cos_lut.argtypes = []
    lib.init_cos_lut()
    own = capi.load()
    capi.check(own)                                   # no usable CUDA device -> raise here, not later

    def to_ref(handle):
        return ctypes.cast(handle, ref_ptr)

    def to_own(handle):
        return ctypes.cast(handle, capi.TensorP)

    def _numpy_to_ctensor(self, arr, dtype):
        """Handle for an operand: a DeviceArray is borrowed (one more reference), a host array is uploaded.
        Released by the caller's free_tensor, as in the reference."""
        if isinstance(arr, DeviceArray):
            own.tops_retain(arr.handle)
            return to_ref(arr.handle)
        dev = DeviceArray.from_numpy(np.ascontiguousarray(arr), dtype, own)
        handle, dev.handle = dev.handle, None
        return to_ref(handle)

    def _ctensor_to_numpy(self, c_tensor, dtype):
        """Adopt the output without copying; the caller's free_tensor drops its own reference."""
        handle = to_own(c_tensor)
        own.tops_retain(handle)
        return DeviceArray(handle, dtype, own)

    def _shape(t):
        return tuple(t.data.shape)

    def _output(shape, dtype):
        arr, nd = capi.shape_array(shape)
        handle = lib.tops_create_uninit(arr, nd, ref_nn.DTYPE_MAP[dtype])
        if not handle:
            capi.check(own)
            raise capi.TensorOpsError("output allocation failed")
        return handle

    def _run(self, name, operands, out_shape, out_dtype):
        handles = [self._numpy_to_ctensor(t.data, t.dtype) for t in operands]
        out = _output(out_shape, out_dtype)
        getattr(lib, name)(*handles, out)
        data = self._ctensor_to_numpy(out, out_dtype)
        for h in handles:
            lib.free_tensor(h)
        lib.free_tensor(out)
        capi.check(own)
        return ref_nn.Tensor(*out_shape, dtype=out_dtype, data=data)

    def _execute_unary(self, input_tensor, c_func_name):
        out_dtype = self.dtype if self.dtype else input_tensor.dtype
        return _run(self, c_func_name, [input_tensor], _shape(input_tensor), out_dtype)

    def _execute_binary(self, input_a, input_b, c_func_name):
        try:
            out_shape = np.broadcast_shapes(_shape(input_a), _shape(input_b))
        except ValueError:
            print(f"Broadcasting error: {input_a.size} vs {input_b.size}")
            raise
        if self.dtype:
            out_dtype = self.dtype
        else:       # promotion over the storage types, as nn/__init__.py:221-226 does
            res = np.result_type(ref_nn.DTYPE_TO_NUMPY[input_a.dtype], ref_nn.DTYPE_TO_NUMPY[input_b.dtype])
            out_dtype = ref_nn.NUMPY_TO_DTYPE.get(res.type, "float32")
        return _run(self, c_func_name, [input_a, input_b], out_shape, out_dtype)

    def _execute_ternary(self, in_a, in_b, in_c, c_func_name):
        try:
            out_shape = np.broadcast_shapes(_shape(in_a), _shape(in_b), _shape(in_c))
        except ValueError:
            print(f"Broadcasting error in ternary op: {in_a.size}, {in_b.size}, {in_c.size}")
            raise
        return _run(self, c_func_name, [in_a, in_b, in_c], out_shape, self.dtype if self.dtype else "float32")

    ops = ref_nn.Ops
    ops._lib = lib
    ops._lib_initialized = True
    ops._numpy_to_ctensor = _numpy_to_ctensor
    ops._ctensor_to_numpy = _ctensor_to_numpy
    ops._execute_unary = _execute_unary
    ops._execute_binary = _execute_binary
    ops._execute_ternary = _execute_ternary
    return lib
