"""Golden vectors generated from the reference's own compiled C library (tests/golden/make_golden.py):
the CPU oracle must reproduce every one of them bit for bit (this is the oracle's pin on machines
without the reference), and so must the CUDA library.  Softmax alone is compared to 1e-6 relative on
the GPU (its parallel sum adds in a different order)."""
import json
import os

import numpy as np
import pytest

from datagen import assert_same_codes, to_f64

HERE = os.path.dirname(os.path.abspath(__file__))
with open(os.path.join(HERE, "golden", "hot_path.json")) as _f:
    MANIFEST = json.load(_f)
ARRAYS = np.load(os.path.join(HERE, "golden", "hot_path.npz"))
CASES = MANIFEST["cases"]


def _run(backend, case):
    ins = [None if k is None else ARRAYS[k] for k in case["inputs"]]
    p = case["params"]
    op = case["op"]
    if op in ("relu", "abs", "cos"):
        return backend.unary(op, ins[0], p["x_dt"], p["out_dt"])
    if op in ("add", "sub", "mul", "div"):
        return backend.binary(op, ins[0], p["a_dt"], ins[1], p["b_dt"], p["out_dt"])
    if op == "quantize":
        return backend.quantize(ins[0], p["x_dt"], ins[1], p["s_dt"], ins[2], p["z_dt"], p["out_dt"], axis=p["axis"])
    if op == "dequantize":
        return backend.dequantize(ins[0], p["x_dt"], ins[1], p["s_dt"], ins[2], p["z_dt"], p["out_dt"])
    if op == "conv2d":
        return backend.conv2d(ins[0], p["x_dt"], ins[1], p["w_dt"], ins[2], p["b_dt"], p["out_dt"], tuple(p["pads"]),
                              tuple(p["strides"]), tuple(p["dilations"]), p["group"])
    if op == "max_pool":
        return backend.max_pool(ins[0], p["x_dt"], p["out_dt"], tuple(p["kernel"]), tuple(p["pads"]), tuple(p["strides"]),
                                tuple(p["dilations"]))
    if op == "gemm":
        return backend.gemm(ins[0], p["a_dt"], ins[1], p["b_dt"], ins[2], p["c_dt"], p["out_dt"], p["alpha"], p["beta"],
                            p["transA"], p["transB"])
    if op == "softmax":
        return backend.softmax(ins[0], p["x_dt"], p["out_dt"], p["axis"])
    raise AssertionError(op)


def _ids(case):
    return f"{case['id']}-{case['op']}"


@pytest.mark.parametrize("case", CASES, ids=_ids)
def test_oracle_reproduces_golden_vectors(port, case):
    want = ARRAYS[f"c{case['id']}_out"]
    assert_same_codes(_run(port, case), want, case["params"]["out_dt"], _ids(case))


@pytest.mark.gpu
@pytest.mark.parametrize("case", CASES, ids=_ids)
def test_cuda_library_reproduces_golden_vectors(case):
    import gpu_ops
    want = ARRAYS[f"c{case['id']}_out"]
    got = _run(gpu_ops, case)
    out_dt = case["params"]["out_dt"]
    if case["op"] == "softmax":
        g, w = to_f64(got, out_dt), to_f64(want, out_dt)
        ulp = {"float32": 2.0 ** -23, "float16": 2.0 ** -10}[out_dt]
        step = {"float32": 2.0 ** -149, "float16": 2.0 ** -24}[out_dt]       # one step below the normal range
        assert np.all(np.abs(g - w) <= (1e-6 + ulp) * np.abs(w) + step + 1e-45)
    else:
        assert_same_codes(got, want, out_dt, _ids(case))


# ---- Cast, Clip, AveragePool, GlobalAveragePool, BatchNormalization (tests/golden/make_adjacent_golden.py) --------------
with open(os.path.join(HERE, "golden", "adjacent_ops.json")) as _f:
    ADJ_CASES = json.load(_f)
ADJ_ARRAYS = np.load(os.path.join(HERE, "golden", "adjacent_ops.npz"))


def _run_adjacent(backend, case):
    ins = [None if k is None else ADJ_ARRAYS[k] for k in case["inputs"]]
    p, op = case["params"], case["op"]
    if op == "cast":
        return backend.cast(ins[0], p["x_dt"], p["out_dt"])
    if op == "clip":
        return backend.clip(ins[0], p["x_dt"], ins[1], p["b_dt"], ins[2], p["b_dt"], p["out_dt"])
    if op == "average_pool":
        return backend.average_pool(ins[0], p["x_dt"], p["out_dt"], tuple(p["kernel"]), tuple(p["pads"]), tuple(p["strides"]),
                                    tuple(p["dilations"]), p["count_include_pad"])
    if op == "global_average_pool":
        return backend.global_average_pool(ins[0], p["x_dt"], p["out_dt"])
    if op == "batch_norm":
        return backend.batch_norm(ins[0], p["x_dt"], ins[1], ins[2], ins[3], ins[4], p["p_dt"], p["out_dt"], p["epsilon"])
    raise AssertionError(op)


@pytest.mark.parametrize("case", ADJ_CASES, ids=_ids)
def test_oracle_reproduces_adjacent_golden_vectors(port, case):
    assert_same_codes(_run_adjacent(port, case), ADJ_ARRAYS[f"c{case['id']}_out"], case["params"]["out_dt"], _ids(case))


@pytest.mark.gpu
@pytest.mark.parametrize("case", ADJ_CASES, ids=_ids)
def test_cuda_library_reproduces_adjacent_golden_vectors(case):
    import gpu_ops
    assert_same_codes(_run_adjacent(gpu_ops, case), ADJ_ARRAYS[f"c{case['id']}_out"], case["params"]["out_dt"], _ids(case))


# ---- Max / Min / Pow, one-line unary operators, MatMul, DynamicQuantizeLinear (tests/golden/make_family_golden.py) ------
with open(os.path.join(HERE, "golden", "family_ops.json")) as _f:
    FAM_CASES = json.load(_f)
FAM_ARRAYS = np.load(os.path.join(HERE, "golden", "family_ops.npz"))
# operators whose expression consists of exactly rounded steps: identical codes on every implementation
FAM_EXACT = {"max", "min", "matmul", "dynamic_quantize"} | {"unary:" + n for n in ("neg", "reciprocal", "ceil", "floor", "sqrt", "round", "softsign", "hard_swish")}


def _run_family(backend, case):
    ins = [FAM_ARRAYS[k] for k in case["inputs"]]
    p, op = case["params"], case["op"]
    if op in ("max", "min", "pow"):
        return (backend.binary(op, ins[0], p["a_dt"], ins[1], p["b_dt"], p["out_dt"]),)
    if op.startswith("unary:"):
        return (backend.unary_math(op[6:], ins[0], p["x_dt"], p["out_dt"]),)
    if op == "matmul":
        return (backend.matmul(ins[0], p["a_dt"], ins[1], p["b_dt"], p["out_dt"]),)
    if op == "dynamic_quantize":
        return tuple(backend.dynamic_quantize_linear(ins[0], p["x_dt"]))
    raise AssertionError(op)


def _family_out_dtypes(case):
    return ("uint8", "float32", "uint8") if case["op"] == "dynamic_quantize" else (case["params"]["out_dt"],)


@pytest.mark.parametrize("case", FAM_CASES, ids=_ids)
def test_oracle_reproduces_family_golden_vectors(port, case):
    """The oracle calls the same glibc functions as the reference: identical codes for every operator."""
    for k, (got, dt) in enumerate(zip(_run_family(port, case), _family_out_dtypes(case))):
        assert_same_codes(got, FAM_ARRAYS[f"c{case['id']}_out{k}"], dt, _ids(case))


@pytest.mark.gpu
@pytest.mark.parametrize("case", FAM_CASES, ids=_ids)
def test_cuda_library_reproduces_family_golden_vectors(case):
    import gpu_ops
    for k, (got, dt) in enumerate(zip(_run_family(gpu_ops, case), _family_out_dtypes(case))):
        want = FAM_ARRAYS[f"c{case['id']}_out{k}"]
        if case["op"] in FAM_EXACT:
            assert_same_codes(got, want, dt, _ids(case))
        elif dt.startswith("int") or dt.startswith("uint"):      # a value at a .5 tie may round either way
            assert np.abs(got.astype(np.int64) - want.astype(np.int64)).max() <= 1
        else:                                                   # CUDA libm against glibc: 2 ulp of the output type
            g, w = to_f64(got, dt), to_f64(want, dt)
            ulp = {"float32": 2.0 ** -23, "float64": 2.0 ** -52, "float16": 2.0 ** -10, "bfloat16": 2.0 ** -7}[dt]
            with np.errstate(invalid="ignore"):
                ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= 2 * ulp * np.abs(w) + 2.0 ** -50)
            assert ok.all(), _ids(case)
