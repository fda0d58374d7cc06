"""The drop-in boundary exercised the way the reference itself uses it.

1. Raw ctypes, exactly the steps of the reference's marshalling helpers (nn/__init__.py:305-344): create_tensor,
   ``ctypes.memmove`` into ``contents.data``, the operator, ``from_address`` read-back, free_tensor -- under
   ``tops_set_memory_mode(1)`` (managed memory), against the oracle.
2. The reference's own, unmodified ``nn/__init__.py`` and ``nn/Operators.py`` (staged by ``make -C oracle refpy``
   into the ignored directory oracle/_ref/nn; skipped when absent) driving the library found as
   ``./tensor_ops.so``: (i) in managed mode with nothing patched, (ii) resident, after
   ``onnx_translator_b200.reference_shim.install(nn)``.  Each runs in a child process, because the reference
   loads its library relative to the working directory and keeps it in a class attribute.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np
import pytest

from reference_python_driver import inputs

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
STAGED = os.path.join(ROOT, "oracle", "_ref")


class _CTensor(ctypes.Structure):                     # the reference's CTensor (nn/__init__.py:9-17)
    _fields_ = [("data", ctypes.c_void_p), ("shape", ctypes.POINTER(ctypes.c_int)), ("ndim", ctypes.c_int),
                ("size", ctypes.c_size_t), ("dtype", ctypes.c_int)]


class _CConvParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("group", ctypes.c_int)]


class _CPoolParams(ctypes.Structure):
    _fields_ = [("pads", ctypes.POINTER(ctypes.c_int)), ("strides", ctypes.POINTER(ctypes.c_int)),
                ("dilations", ctypes.POINTER(ctypes.c_int)), ("kernel_shape", ctypes.POINTER(ctypes.c_int))]


_CODES = {"float32": 4, "int8": 7}


@pytest.fixture()
def managed_lib():
    from onnx_translator_b200 import capi
    capi.load()
    lib = ctypes.CDLL(capi.LIB_PATH)                  # a plain handle: only what the reference declares is declared
    lib.create_tensor.restype = ctypes.POINTER(_CTensor)
    lib.create_tensor.argtypes = [ctypes.POINTER(ctypes.c_int), ctypes.c_int, ctypes.c_int]
    lib.free_tensor.argtypes = [ctypes.POINTER(_CTensor)]
    lib.tops_last_error_message.restype = ctypes.c_char_p
    lib.tops_set_memory_mode(1)
    yield lib
    lib.tops_set_memory_mode(0)


def _to_c(lib, arr, dtype):                            # nn/__init__.py:305-323
    arr = np.ascontiguousarray(arr)
    shape = (ctypes.c_int * arr.ndim)(*arr.shape)
    t = lib.create_tensor(shape, arr.ndim, _CODES[dtype])
    assert t, lib.tops_last_error_message()
    ctypes.memmove(t.contents.data, arr.ctypes.data, arr.size * arr.itemsize)
    return t


def _new(lib, shape, dtype):
    arr = (ctypes.c_int * len(shape))(*shape)
    t = lib.create_tensor(arr, len(shape), _CODES[dtype])
    assert t, lib.tops_last_error_message()
    return t


def _to_numpy(t, np_dtype):                            # nn/__init__.py:325-344
    c = t.contents
    shape = [c.shape[i] for i in range(c.ndim)]
    nbytes = c.size * np.dtype(np_dtype).itemsize
    return np.frombuffer((ctypes.c_byte * nbytes).from_address(c.data), dtype=np_dtype).reshape(shape).copy()


def _ints(v):
    return ctypes.cast((ctypes.c_int * len(v))(*v), ctypes.POINTER(ctypes.c_int))


def test_reference_marshalling_steps_work_on_managed_memory(managed_lib, port):
    lib, d = managed_lib, inputs()
    f32 = "float32"
    P = ctypes.POINTER(_CTensor)

    def call(fn, operands, out_shape, out_dt, extra=()):
        handles = [_to_c(lib, a, dt) if a is not None else P() for a, dt in operands]
        out = _new(lib, out_shape, out_dt)
        assert not _to_numpy(out, np.float32 if out_dt == f32 else np.int8).any()       # create_tensor zero-fills, like calloc
        getattr(lib, fn)(*handles, out, *extra)
        got = _to_numpy(out, np.float32 if out_dt == f32 else np.int8)
        for h in handles:
            if h:
                lib.free_tensor(h)
        lib.free_tensor(out)
        assert lib.tops_last_error() == 0, lib.tops_last_error_message()
        return got

    same = lambda got, want: np.array_equal(np.ascontiguousarray(got).view(np.uint8), np.ascontiguousarray(want).view(np.uint8))
    # Add: the reference broadcasts on the host and passes equal-size operands (nn/__init__.py:213-236)
    a, b = np.broadcast_arrays(d["a"], d["b"])
    assert same(call("add_forward", [(a, f32), (b, f32)], a.shape, f32), port.binary("add", a, f32, np.ascontiguousarray(b), f32, f32))
    # QuantizeLinear with scale and zero point pre-broadcast to X's shape, as _execute_ternary passes them
    x, s, z = np.broadcast_arrays(d["c"], d["q_scale"].reshape(1, 16, 1, 1), d["q_zero"].reshape(1, 16, 1, 1))
    want = port.quantize(d["c"], f32, d["q_scale"].reshape(1, 16, 1, 1), f32, d["q_zero"].reshape(1, 16, 1, 1), "int8", "int8")
    assert same(call("quantize_linear_forward", [(x, f32), (s, f32), (z, "int8")], x.shape, "int8"), want)
    # Conv, MaxPool, Gemm, Softmax with the reference's attribute structs
    keep = [_ints([1, 1, 1, 1]), _ints([1, 1]), _ints([1, 1])]
    prm = _CConvParams(keep[0], keep[1], keep[2], 1)
    conv = call("conv2d_forward", [(d["x"], f32), (d["w"], f32), (d["wb"], f32)], (2, 8, 16, 16), f32, (ctypes.byref(prm),))
    want_conv = port.conv2d(d["x"], f32, d["w"], f32, d["wb"], f32, f32, (1, 1, 1, 1), (1, 1), (1, 1), 1)
    assert same(conv, want_conv)
    keep2 = [_ints([0, 0, 0, 0]), _ints([2, 2]), _ints([1, 1]), _ints([2, 2])]
    pool_prm = _CPoolParams(keep2[0], keep2[1], keep2[2], keep2[3])
    pool = call("max_pool_forward", [(conv, f32)], (2, 8, 8, 8), f32, (ctypes.byref(pool_prm),))
    assert same(pool, port.max_pool(want_conv, f32, f32, (2, 2), (0, 0, 0, 0), (2, 2)))
    lib.gemm_forward.argtypes = [P, P, P, P, ctypes.c_float, ctypes.c_float, ctypes.c_int, ctypes.c_int]
    gemm = call("gemm_forward", [(d["ga"], f32), (d["gb"], f32), (d["gc"].reshape(1, -1), f32)], (5, 10), f32, (0.5, 2.0, 0, 1))
    want_gemm = port.gemm(d["ga"], f32, d["gb"], f32, d["gc"], f32, f32, 0.5, 2.0, 0, 1)
    assert same(gemm, want_gemm)
    soft = call("softmax_forward", [(gemm, f32)], (5, 10), f32, (ctypes.c_int(1),))
    assert np.allclose(soft, port.softmax(want_gemm, f32, f32, 1), rtol=1e-6, atol=0)


def _oracle_results(port):
    """The same operator calls as tests/reference_python_driver.py:run, evaluated by the oracle."""
    d, f32 = inputs(), "float32"
    w = {}
    for name in ("add", "sub", "mul", "div"):
        w[name] = port.binary(name, d["a"], f32, d["b"], f32, f32)
        w[name + "_i8"] = port.binary(name, d["ai"], "int8", d["bi"], "int8", "int8")
    w["relu"] = port.unary("relu", d["a"], f32, f32)
    w["abs"] = port.unary("abs", d["ai"], "int8", "int8")
    w["cos"] = port.unary("cos", d["c"], f32, f32)
    w["quant"] = port.quantize(d["c"], f32, d["q_scale"], f32, d["q_zero"], "int8", "int8", axis=1)
    w["dequant"] = port.dequantize(w["quant"], "int8", d["q_scale"].reshape(16, 1, 1), f32, d["q_zero"].reshape(16, 1, 1), "int8", f32)
    w["conv"] = port.conv2d(d["x"], f32, d["w"], f32, d["wb"], f32, f32, (1, 1, 1, 1), (1, 1), (1, 1), 1)
    w["pool"] = port.max_pool(port.unary("relu", w["conv"], f32, f32), f32, f32, (2, 2), (0, 0, 0, 0), (2, 2))
    w["flat"] = w["pool"].reshape(2, -1)
    w["gemm"] = port.gemm(d["ga"], f32, d["gb"], f32, d["gc"], f32, f32, 0.5, 2.0, 0, 1)
    w["softmax"] = port.softmax(w["gemm"], f32, f32, 1)
    return w


@pytest.mark.parametrize("mode", ["managed", "resident"])
def test_the_references_own_operator_classes_drive_the_library(mode, port, tmp_path):
    from onnx_translator_b200 import capi
    if not os.path.exists(os.path.join(STAGED, "nn", "Operators.py")):
        pytest.skip("the reference's nn package is not staged (make -C oracle refpy needs the reference checkout)")
    capi.load()
    os.symlink(capi.LIB_PATH, tmp_path / "tensor_ops.so")          # where nn/__init__.py:150 looks for it
    out = tmp_path / "out.npz"
    driver = os.path.join(ROOT, "tests", "reference_python_driver.py")
    res = subprocess.run([sys.executable, driver, mode, STAGED, ROOT, str(out)], cwd=tmp_path, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-4000:]
    got = np.load(out)
    want = _oracle_results(port)
    assert set(got.files) == set(want)
    for name, w in want.items():
        g = got[name]
        assert g.shape == w.shape and g.dtype == w.dtype, name
        if name == "softmax":
            assert np.allclose(g, w, rtol=1e-6, atol=0), name
        else:
            assert np.array_equal(g.view(np.uint8), np.ascontiguousarray(w).view(np.uint8)), name
