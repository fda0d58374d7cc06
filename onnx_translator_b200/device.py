"""DeviceArray: a tensor that lives in GPU memory between operators.

It owns one reference to a library ``Tensor`` (include/tensor_ops_b200.h) and offers the few
ndarray attributes the reference's operator classes touch on ``Tensor.data`` (``shape``, ``ndim``,
``size``, ``reshape``; nn/Operators.py:439-445, 640-645), plus explicit transfers.  Converting it
with ``numpy.asarray`` downloads the contents.
"""
from __future__ import annotations

import ctypes
from typing import Optional, Sequence

import numpy as np

from . import capi


class DeviceArray:
    __slots__ = ("handle", "dtype_name", "_lib", "__weakref__")

    def __init__(self, handle, dtype_name: str, lib=None):
        if not handle:
            raise capi.TensorOpsError("null tensor handle")
        self.handle = handle                 # POINTER(CTensor); this object holds one reference
        self.dtype_name = dtype_name
        self._lib = lib or capi.load()

    # -- construction ------------------------------------------------------------------------
    @classmethod
    def empty(cls, shape: Sequence[int], dtype_name: str, zero: bool = False, lib=None) -> "DeviceArray":
        lib = lib or capi.load()
        arr, nd = capi.shape_array(shape)
        make = lib.create_tensor if zero else lib.tops_create_uninit
        handle = make(arr, nd, capi.DTYPE_MAP[dtype_name])
        if not handle:
            capi.check(lib)
            raise capi.TensorOpsError("tensor allocation failed")
        return cls(handle, dtype_name, lib)

    @classmethod
    def from_numpy(cls, array, dtype_name: Optional[str] = None, lib=None) -> "DeviceArray":
        """Upload a host array.  ``dtype_name`` defaults from the numpy dtype (uint16 means
        bfloat16 codes, as in the reference's tables)."""
        if dtype_name is None:
            dtype_name = capi.NUMPY_TO_DTYPE.get(np.asarray(array).dtype.type, "float32")
        host = np.ascontiguousarray(array, dtype=capi.DTYPE_TO_NUMPY[dtype_name])
        out = cls.empty(host.shape, dtype_name, lib=lib)
        if host.nbytes:
            rc = out._lib.tops_upload(out.handle, host.ctypes.data, host.nbytes)
            if rc:
                capi.check(out._lib)
            # pageable memory: the copy has been staged when the call returns; pinned memory
            # callers (bench) keep their buffer alive themselves
        return out

    # -- ndarray-like surface ----------------------------------------------------------------------
    @property
    def shape(self):
        c = self.handle.contents
        return tuple(c.shape[i] for i in range(c.ndim))

    @property
    def ndim(self) -> int:
        return self.handle.contents.ndim

    @property
    def size(self) -> int:
        return self.handle.contents.size

    @property
    def dtype(self):
        return np.dtype(capi.DTYPE_TO_NUMPY[self.dtype_name])

    @property
    def nbytes(self) -> int:
        return self.size * self.dtype.itemsize

    @property
    def data_ptr(self) -> int:
        return self.handle.contents.data or 0

    # -- zero-copy hand-over to frameworks ---------------------------------------------------------------
    _TYPESTR = {"float32": "<f4", "float64": "<f8", "float16": "<f2", "int8": "|i1", "uint8": "|u1", "int4": "|i1", "int16": "<i2",
                "int32": "<i4", "int64": "<i8", "bfloat16": "<u2", "float8_e4m3": "|u1", "float8_e5m2": "|u1", "bool": "|u1"}

    @property
    def __cuda_array_interface__(self):
        """The CUDA array interface (version 2): lets torch / cupy / numba view the memory without a copy.  Types numpy
        has no name for travel as their storage codes (bfloat16 as uint16, float8 as uint8)."""
        return {"shape": self.shape, "typestr": self._TYPESTR[self.dtype_name], "data": (self.data_ptr, False), "version": 2}

    def as_torch(self):
        """A torch tensor over the same device memory (no copy); it keeps this array alive.  Work enqueued on the
        library's stream must be ordered before torch touches it: run torch under
        ``torch.cuda.ExternalStream(lib.tops_get_stream())`` or call ``tops_sync`` first."""
        import torch
        device = self._lib.tops_get_device()
        t = torch.as_tensor(self, device=torch.device("cuda", device))
        if self.dtype_name == "bfloat16":
            t = t.view(torch.bfloat16)                 # the interface carried the codes as 16-bit integers
        t._tops_owner = self
        return t

    def reshape(self, *shape) -> "DeviceArray":
        """Zero-copy view with a new shape (one -1 allowed)."""
        if len(shape) == 1 and isinstance(shape[0], (tuple, list)):
            shape = tuple(shape[0])
        shape = [int(s) for s in shape]
        if shape.count(-1) == 1:
            known = 1
            for s in shape:
                if s != -1:
                    known *= s
            shape[shape.index(-1)] = self.size // known if known else 0
        arr, nd = capi.shape_array(shape)
        handle = self._lib.tops_view(self.handle, arr, nd)
        if not handle:
            capi.check(self._lib)
            raise capi.TensorOpsError("reshape failed")
        return DeviceArray(handle, self.dtype_name, self._lib)

    def rows(self, begin: int, count: int) -> "DeviceArray":
        """View of rows [begin, begin+count) along dimension 0."""
        handle = self._lib.tops_slice_rows(self.handle, int(begin), int(count))
        if not handle:
            capi.check(self._lib)
            raise capi.TensorOpsError("row slice failed")
        return DeviceArray(handle, self.dtype_name, self._lib)

    def numpy(self) -> np.ndarray:
        out = np.empty(self.shape, dtype=capi.DTYPE_TO_NUMPY[self.dtype_name])
        if out.nbytes:
            rc = self._lib.tops_download(self.handle, out.ctypes.data, out.nbytes)
            if rc:
                capi.check(self._lib)
        return out

    def __array__(self, dtype=None, copy=None):
        out = self.numpy()
        return out.astype(dtype) if dtype is not None else out

    def astype(self, dtype, copy=False):
        return self.numpy().astype(dtype, copy=copy)

    def __len__(self):
        return self.shape[0]

    def __repr__(self):
        return f"DeviceArray(shape={self.shape}, dtype={self.dtype_name})"

    def __del__(self):
        try:
            if self.handle:
                self._lib.free_tensor(self.handle)
                self.handle = None
        except Exception:
            pass


def is_device(obj) -> bool:
    return isinstance(obj, DeviceArray)
