"""CPU-side checks of the C-ABI library: it loads, exports every symbol the public header
declares, the ctypes table covers the header, and the host-only pieces (broadcast planner)
behave.  No kernel is launched here."""
import ctypes
import os
import re
import subprocess

import numpy as np
import pytest

from onnx_translator_b200 import capi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "tensor_ops_b200.h")


def _declared_functions():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    names = re.findall(r"^[A-Za-z_][A-Za-z0-9_ \*]*?\b([a-z_0-9]+)\s*\(", text, flags=re.M)
    return sorted(set(n for n in names if n not in ("defined",)))


@pytest.fixture(scope="module")
def lib():
    if not os.path.exists(capi.LIB_PATH):
        from onnx_translator_b200 import build
        build.build()
    return capi.load()


def test_header_declares_the_reference_entry_points():
    names = _declared_functions()
    for must in ("create_tensor", "free_tensor", "init_cos_lut", "relu_forward", "cos_forward", "abs_forward",
                 "add_forward", "sub_forward", "mul_forward", "div_forward", "quantize_linear_forward",
                 "dequantize_linear_forward", "conv2d_forward", "max_pool_forward", "gemm_forward",
                 "softmax_forward", "flatten_forward", "reshape_forward"):
        assert must in names


def test_library_exports_every_declared_symbol(lib):
    exported = subprocess.run(["nm", "-D", "--defined-only", capi.LIB_PATH], capture_output=True, text=True, check=True).stdout
    exported = set(line.split()[-1] for line in exported.splitlines() if " T " in line)
    for name in _declared_functions():
        assert name in exported, f"{name} is declared in the header but not exported"
        assert name in capi.SIGNATURES, f"{name} has no ctypes signature"
    assert set(capi.SIGNATURES) <= set(_declared_functions())


def test_struct_layouts_match_the_reference_abi():
    # x86-64: void*, int*, int (+pad), size_t, int (+pad) -> 40 bytes (tensor_ops/tensor_ops.h:28-34)
    assert ctypes.sizeof(capi.CTensor) == 40
    assert capi.CTensor.data.offset == 0 and capi.CTensor.shape.offset == 8
    assert capi.CTensor.ndim.offset == 16 and capi.CTensor.size.offset == 24 and capi.CTensor.dtype.offset == 32
    assert ctypes.sizeof(capi.CConvParams) == 32 and ctypes.sizeof(capi.CPoolParams) == 32
    assert [capi.DTYPE_MAP[k] for k in ("float8_e4m3", "float8_e5m2", "float16", "bfloat16", "float32", "float64",
                                        "int4", "int8", "uint8", "int16", "int32", "int64")] == list(range(12))
    assert capi.load().tops_dtype_size(capi.DTYPE_MAP["bfloat16"]) == 2


def _plan(lib, out_shape, in_shape):
    o = (ctypes.c_int * max(len(out_shape), 1))(*out_shape)
    i = (ctypes.c_int * max(len(in_shape), 1))(*in_shape)
    nd, flat = ctypes.c_int(), ctypes.c_int()
    sizes = (ctypes.c_uint * 16)()
    strides = (ctypes.c_int * 16)()
    ok = lib.tops_debug_plan_broadcast(o, len(out_shape), i, len(in_shape), ctypes.byref(nd), sizes, strides, ctypes.byref(flat))
    return ok, nd.value, list(sizes[:nd.value]), list(strides[:nd.value]), flat.value


@pytest.mark.parametrize("out_shape,in_shape", [
    ((64, 512, 1024), (1, 512, 1)), ((64, 512, 1024), (1024,)), ((64, 512, 1024), (64, 512, 1024)),
    ((10, 10, 10), (10, 1)), ((4, 3, 16), (16,)), ((2, 16, 14, 14), (16, 1, 1)), ((5,), (1,)), ((6, 7), (1, 1)),
    ((2, 3, 4, 5, 6), (3, 1, 5, 1)), ((4, 3, 5), (4, 1, 5)), ((3, 2, 2, 2, 2, 2, 3), (1, 2, 1, 2, 1, 2, 1)),
])
def test_broadcast_plan_reproduces_numpy_indexing(lib, out_shape, in_shape):
    ok, nd, sizes, strides, flat = _plan(lib, out_shape, in_shape)
    assert ok
    total = int(np.prod(out_shape))
    src = np.arange(int(np.prod(in_shape))).reshape(in_shape)
    want = np.broadcast_to(src, out_shape).reshape(-1)
    if flat:
        assert np.prod(in_shape) == total
        return
    assert int(np.prod(sizes)) == total and nd <= 16
    idx = np.arange(total)
    off = np.zeros(total, dtype=np.int64)
    for d in range(nd - 1, -1, -1):
        off += (idx % sizes[d]) * strides[d]
        idx //= sizes[d]
    assert np.array_equal(off, want)


def test_broadcast_plan_collapses_the_benchmark_shapes(lib):
    assert _plan(lib, (64, 512, 1024), (1, 512, 1))[1:4] == (3, [64, 512, 1024], [0, 1, 0])
    assert _plan(lib, (64, 512, 1024), (1024,))[1:4] == (2, [64 * 512, 1024], [0, 1])
    assert _plan(lib, (256, 64, 56, 56), (64, 1, 1))[1:4] == (3, [256, 64, 3136], [0, 1, 0])
    assert _plan(lib, (8, 4), (1,))[1:4] == (1, [32], [0])


def test_broadcast_plan_rejects_incompatible_shapes(lib):
    assert _plan(lib, (3, 4), (5,))[0] == 0
    assert _plan(lib, (3, 4), (2, 3, 4))[0] == 0
    assert _plan(lib, (3, 4), (2, 1, 4))[0] == 0
    # equal element counts pair up flat, whatever the shapes (the reference only compares sizes)
    assert _plan(lib, (3, 4), (3, 1, 4))[4] == 1


def test_missing_library_is_a_loud_error(tmp_path):
    with pytest.raises(capi.TensorOpsError):
        capi.load(str(tmp_path / "absent.so"))


def test_no_gpu_means_errors_not_a_cpu_path(lib):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    shape = (ctypes.c_int * 1)(4)
    lib.tops_clear_error()
    assert not lib.create_tensor(shape, 1, capi.DTYPE_MAP["float32"])
    assert lib.tops_last_error() != 0
    lib.tops_clear_error()
    from onnx_translator_b200 import nn
    from onnx_translator_b200.nn import Operators
    nn.Ops._lib = None
    node = Operators.RELU([], [], dtype="float32")              # constructing a node needs no GPU ...
    with pytest.raises(capi.TensorOpsError):                     # ... running it without one fails loudly
        node.forward(nn.Tensor(4, dtype="float32"))
    lib.tops_clear_error()
