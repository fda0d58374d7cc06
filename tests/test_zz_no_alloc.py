"""The allocation-free convolution entry point (tops_conv2d_forward_noalloc).

It exists for callers that cannot let this library take GPU memory from the driver or the CUDA pool
while they run (a process with its own arena allocator or a fixed memory budget): its scratch is a
fixed array inside the library image.  Here it is called through the C ABI twice in a row, with
different shapes and data, and each result must equal conv2d_forward's bit for bit (both run the
same tensor-core kernel; only where the scratch lives differs).  The second call is smaller than
the first, so stale bytes of the first call sit right behind its scratch region.  Problems whose
scratch exceeds the fixed size must be refused with a clear error.
This file is collected last on purpose.
"""
import ctypes

import numpy as np
import pytest

from datagen import from_f64

pytestmark = pytest.mark.gpu


def _params(pads, strides, dil, group=1):
    from onnx_translator_b200.capi import CConvParams
    keep = [(ctypes.c_int * len(v))(*v) for v in (pads, strides, dil)]
    prm = CConvParams(*[ctypes.cast(k, ctypes.POINTER(ctypes.c_int)) for k in keep], group)
    return prm, keep


def _both(lib, x, w, b, dt, out_dt, pads, dil):
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    n, _, h, wd = x.shape
    m, _, kh, kw = w.shape
    oh = h + pads[0] + pads[2] - dil[0] * (kh - 1)
    ow = wd + pads[1] + pads[3] - dil[1] * (kw - 1)
    xd, wdv = DeviceArray.from_numpy(x, dt), DeviceArray.from_numpy(w, dt)
    bd = None if b is None else DeviceArray.from_numpy(b, "float32")
    prm, keep = _params(pads, (1, 1), dil)
    fill = 0x7F if out_dt != "float32" else 0
    y_pool = DeviceArray.from_numpy(np.full((n, m, oh, ow), fill, capi.DTYPE_TO_NUMPY[out_dt]), out_dt)
    y_fixed = DeviceArray.from_numpy(np.full((n, m, oh, ow), fill, capi.DTYPE_TO_NUMPY[out_dt]), out_dt)
    before = lib.tops_tensor_core_launches()
    lib.conv2d_forward(xd.handle, wdv.handle, bd.handle if bd else None, y_pool.handle, ctypes.byref(prm))
    lib.tops_conv2d_forward_noalloc(xd.handle, wdv.handle, bd.handle if bd else None, y_fixed.handle, ctypes.byref(prm))
    capi.check(lib)
    assert lib.tops_tensor_core_launches() == before + 2, "both calls must run the tensor-core kernel"
    return y_pool.numpy(), y_fixed.numpy()


def test_fixed_scratch_convolution_matches_the_pool_one_on_two_calls_in_a_row():
    from onnx_translator_b200 import capi
    lib = capi.load()
    rng = np.random.default_rng(2024)
    # call 1: 4 x 64 x 28 x 28, 128 filters 3x3, bias, bfloat16 in / float32 out
    x1 = from_f64(rng.normal(0, 1, (4, 64, 28, 28)), "bfloat16")
    w1 = from_f64(rng.normal(0, 0.05, (128, 64, 3, 3)), "bfloat16")
    b1 = rng.normal(0, 1, 128).astype(np.float32)
    ref1, got1 = _both(lib, x1, w1, b1, "bfloat16", "float32", (1, 1, 1, 1), (1, 1))
    assert np.array_equal(ref1.view(np.uint32), got1.view(np.uint32))
    assert np.abs(got1).max() > 0
    # call 2, straight after: smaller, other dtype, dilation 2, no bias, 16-bit output
    x2 = from_f64(rng.normal(0, 1, (3, 32, 20, 24)), "float16")
    w2 = from_f64(rng.normal(0, 0.05, (96, 32, 3, 3)), "float16")
    ref2, got2 = _both(lib, x2, w2, None, "float16", "float16", (2, 2, 2, 2), (2, 2))
    assert np.array_equal(ref2.view(np.uint16), got2.view(np.uint16))
    # and the first problem again: same answer as before
    ref3, got3 = _both(lib, x1, w1, b1, "bfloat16", "float32", (1, 1, 1, 1), (1, 1))
    assert np.array_equal(got3.view(np.uint32), got1.view(np.uint32)) and np.array_equal(ref3.view(np.uint32), got1.view(np.uint32))


def test_problems_beyond_the_fixed_scratch_are_refused():
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    cap_in, cap_w = ctypes.c_size_t(), ctypes.c_size_t()
    total = lib.tops_conv2d_noalloc_limits(ctypes.byref(cap_in), ctypes.byref(cap_w))
    assert total == cap_in.value + cap_w.value == 36 << 20
    # padded input 16 x 58 x 58 x 512 x 2 bytes = 55 MB > 32 MiB
    x = DeviceArray.empty((16, 512, 56, 56), "bfloat16")
    w = DeviceArray.empty((64, 512, 3, 3), "bfloat16")
    y = DeviceArray.from_numpy(np.full((16, 64, 56, 56), 5.0, np.float32), "float32")
    prm, keep = _params((1, 1, 1, 1), (1, 1), (1, 1))
    lib.tops_clear_error()
    lib.tops_conv2d_forward_noalloc(x.handle, w.handle, None, y.handle, ctypes.byref(prm))
    assert lib.tops_last_error() == 5
    assert b"exceeds" in lib.tops_last_error_message()
    lib.tops_clear_error()
    assert not y.numpy().any()                      # refused calls leave a zero-filled output
    # stride 2 is outside the tensor-core path: refused as well, not silently handed to another kernel
    x2 = DeviceArray.empty((2, 32, 16, 16), "bfloat16")
    w2 = DeviceArray.empty((64, 32, 3, 3), "bfloat16")
    y2 = DeviceArray.empty((2, 64, 8, 8), "float32")
    prm2, keep2 = _params((1, 1, 1, 1), (2, 2), (1, 1))
    lib.tops_conv2d_forward_noalloc(x2.handle, w2.handle, None, y2.handle, ctypes.byref(prm2))
    assert lib.tops_last_error() == 5
    lib.tops_clear_error()
