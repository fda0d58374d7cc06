"""Child process of tests/test_gpu_reference_python.py: imports the REFERENCE's own ``nn`` package (staged
unmodified under oracle/_ref/nn by ``make -C oracle refpy``) and runs its hot-path operator classes against
the CUDA library, found the way the reference finds its library: ``./tensor_ops.so`` in the working directory
(nn/__init__.py:150).

    python reference_python_driver.py managed|resident <staged dir> <repo root> <out.npz>

managed:  nothing of the reference is touched; the library is switched to managed memory first, so the
          reference's memmove into Tensor.data and its read-back through the pointer work (nn/__init__.py:305-344).
resident: onnx_translator_b200.reference_shim.install(nn) replaces the marshalling helpers; operator results
          stay on the device and feed the next operator without a copy.
"""
import ctypes
import os
import sys

import numpy as np


def inputs():
    """Seeded operands of the thirteen hot-path operators (shared with the parent test)."""
    rng = np.random.default_rng(1234)
    d = {}
    d["a"] = rng.uniform(-100, 100, (2, 16, 8, 8)).astype(np.float32)
    d["b"] = rng.uniform(0.5, 100, (16, 1, 1)).astype(np.float32) * rng.choice([-1, 1], (16, 1, 1)).astype(np.float32)
    d["ai"] = rng.integers(-100, 100, (2, 16, 8, 8)).astype(np.int8)
    d["bi"] = rng.integers(1, 100, (2, 16, 8, 8)).astype(np.int8)
    d["c"] = rng.uniform(-10, 10, (2, 16, 8, 8)).astype(np.float32)
    d["q_scale"] = rng.uniform(0.01, 0.05, 16).astype(np.float32)
    d["q_zero"] = rng.integers(-8, 9, 16).astype(np.int8)
    d["x"] = rng.standard_normal((2, 3, 16, 16)).astype(np.float32)
    d["w"] = rng.normal(0, 0.1, (8, 3, 3, 3)).astype(np.float32)
    d["wb"] = rng.normal(0, 1, 8).astype(np.float32)
    d["ga"] = rng.normal(0, 1, (5, 64)).astype(np.float32)
    d["gb"] = rng.normal(0, 0.1, (10, 64)).astype(np.float32)
    d["gc"] = rng.normal(0, 1, 10).astype(np.float32)
    return d


def run(R, T, d):
    """The operator calls, through whatever ``R`` (an Operators module) and ``T`` (its Tensor class) are."""
    f32 = "float32"
    t = lambda a, dt=f32: T(*a.shape, dtype=dt, data=a)
    out = {}
    keep = lambda name, res: out.__setitem__(name, res["tensor"]) or res["tensor"]
    for name, cls in (("add", R.ADD), ("sub", R.SUB), ("mul", R.MUL), ("div", R.DIV)):
        keep(name, cls([], [], dtype=f32).forward(t(d["a"]), t(d["b"])))
        keep(name + "_i8", cls([], [], dtype="int8").forward(t(d["ai"], "int8"), t(d["bi"], "int8")))
    keep("relu", R.RELU([], [], dtype=f32).forward(t(d["a"])))
    keep("abs", R.ABS([], [], dtype="int8").forward(t(d["ai"], "int8")))
    keep("cos", R.COS([], [], dtype=f32).forward(t(d["c"])))
    q = keep("quant", R.QuantizeLinear([], [], axis=1, dtype="int8").forward(t(d["c"]), t(d["q_scale"]), t(d["q_zero"], "int8")))
    keep("dequant", R.DequantizeLinear([], [], dtype=f32).forward(q, t(d["q_scale"].reshape(16, 1, 1)), t(d["q_zero"].reshape(16, 1, 1), "int8")))
    # a chain, so that in resident mode operator outputs feed operators: conv -> relu -> maxpool -> flatten -> gemm -> softmax
    y = keep("conv", R.Conv([], [], pads=[1, 1, 1, 1], strides=[1, 1], dilations=[1, 1], group=1, dtype=f32).forward(t(d["x"]), t(d["w"]), t(d["wb"])))
    y = R.RELU([], [], dtype=f32).forward(y)["tensor"]
    y = keep("pool", R.MaxPool([], [], kernel_shape=[2, 2], pads=[0, 0, 0, 0], strides=[2, 2], dtype=f32).forward(y))
    keep("flat", R.Flatten([], [], axis=1, dtype=f32).forward(y))
    g = keep("gemm", R.Gemm([], [], alpha=0.5, beta=2.0, transA=0, transB=1, dtype=f32).forward(t(d["ga"]), t(d["gb"]), t(d["gc"])))
    keep("softmax", R.Softmax([], [], axis=1, dtype=f32).forward(g))
    return out


def main():
    mode, staged, root, out_path = sys.argv[1:5]
    sys.path.insert(0, staged)
    sys.path.insert(1, root)
    assert os.path.exists("./tensor_ops.so"), "run from a directory that holds tensor_ops.so"
    if mode == "managed":
        lib = ctypes.CDLL("./tensor_ops.so")
        lib.tops_set_memory_mode(1)
    import nn                                    # the reference's package
    assert os.path.realpath(nn.__file__).startswith(os.path.realpath(staged)), nn.__file__
    from nn import Operators as R
    if mode == "resident":
        from onnx_translator_b200 import reference_shim
        from onnx_translator_b200.device import DeviceArray
        lib = reference_shim.install(nn)
    results = run(R, nn.Tensor, inputs())
    if mode == "resident":
        assert all(isinstance(v.data, DeviceArray) for v in results.values()), "results must stay on the device"
    else:
        assert all(isinstance(v.data, np.ndarray) for v in results.values())
    lib.tops_last_error.restype = ctypes.c_int
    lib.tops_last_error_message.restype = ctypes.c_char_p
    assert lib.tops_last_error() == 0, lib.tops_last_error_message()
    np.savez(out_path, **{k: np.asarray(v.data) for k, v in results.items()})


if __name__ == "__main__":
    main()
