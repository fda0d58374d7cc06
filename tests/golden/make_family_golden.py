"""Generates tests/golden/family_ops.npz + family_ops.json from the reference's OWN C library
(oracle/_ref/tensor_ops_ref.so): Max / Min / Pow, the 25 one-line unary operators, MatMul and
DynamicQuantizeLinear on small seeded inputs.  Run where the reference sources are available:

    python tests/golden/make_family_golden.py
"""
import json
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "tests"))

import oracle  # noqa: E402
from datagen import FLOAT_DTYPES, make  # noqa: E402

def main():
    ref = oracle.HostOracle("ref")
    rng = np.random.default_rng(20240703)
    arrays, cases = {}, []

    def add(op, inputs, params, outs):
        idx = len(cases)
        names = []
        for k, arr in enumerate(inputs):
            arrays[f"c{idx}_in{k}"] = np.ascontiguousarray(arr)
            names.append(f"c{idx}_in{k}")
        outs = outs if isinstance(outs, tuple) else (outs,)
        for k, arr in enumerate(outs):
            arrays[f"c{idx}_out{k}"] = np.ascontiguousarray(arr)
        cases.append({"id": idx, "op": op, "inputs": names, "params": params, "n_out": len(outs)})

    for op in ("max", "min", "pow"):
        for a_dt, b_dt, out_dt in (("float32", "float32", "float32"), ("float16", "float16", "float16"), ("int8", "int8", "int8"),
                                   ("int32", "float16", "float64"), ("bfloat16", "float32", "float32")):
            a, b = make(rng, (5, 7, 6), a_dt), make(rng, (7, 1), b_dt)
            if a_dt == "float32":
                a.reshape(-1)[:6] = [np.nan, 1.0, np.inf, -np.inf, 0.0, -0.0]
                b.reshape(-1)[:2] = [1.0, np.nan]
            add(op, [a, b], {"a_dt": a_dt, "b_dt": b_dt, "out_dt": out_dt}, ref.binary(op, a, a_dt, b, b_dt, out_dt))
    for op in oracle.HostOracle.UNARY_MATH:
        for x_dt, out_dt in (("float32", "float32"), ("float16", "float16"), ("int8", "float32"), ("float64", "float64"), ("bfloat16", "int32")):
            x = make(rng, (9, 11), x_dt, -3, 3) if x_dt in FLOAT_DTYPES else make(rng, (9, 11), x_dt)
            if x_dt == "float32":
                x.reshape(-1)[:9] = [0.0, -0.0, 1.0, -1.0, 0.5, 2.5, np.inf, -np.inf, np.nan]
            add("unary:" + op, [x], {"x_dt": x_dt, "out_dt": out_dt}, ref.unary_math(op, x, x_dt, out_dt))
    for a_dt, b_dt, out_dt, a_shape, b_shape in (("float32", "float32", "float32", (7, 13), (13, 5)), ("float32", "float32", "float32", (3, 2, 7, 13), (13, 5)),
                                                 ("float16", "float16", "float16", (4, 6, 9), (4, 9, 11)), ("bfloat16", "float32", "float32", (2, 1, 6, 8), (1, 3, 8, 4)),
                                                 ("float64", "float64", "float64", (5, 17), (2, 17, 3)), ("int8", "int8", "int32", (3, 5, 12), (12, 7))):
        a, b = make(rng, a_shape, a_dt), make(rng, b_shape, b_dt)
        add("matmul", [a, b], {"a_dt": a_dt, "b_dt": b_dt, "out_dt": out_dt}, ref.matmul(a, a_dt, b, b_dt, out_dt))
    for x_dt, shape in (("float32", (5, 77)), ("float32", (4099,)), ("float16", (3, 40)), ("bfloat16", (130,)), ("float64", (33,)), ("int8", (64,))):
        x = make(rng, shape, x_dt)
        add("dynamic_quantize", [x], {"x_dt": x_dt, "out_dt": "uint8"}, ref.dynamic_quantize_linear(x, x_dt))
    odd = make(rng, (64,), "float32")
    odd[:3] = [np.nan, 1e30, -3.0]
    add("dynamic_quantize", [odd], {"x_dt": "float32", "out_dt": "uint8"}, ref.dynamic_quantize_linear(odd, "float32"))
    np.savez_compressed(os.path.join(HERE, "family_ops.npz"), **arrays)
    with open(os.path.join(HERE, "family_ops.json"), "w") as f:
        json.dump(cases, f, indent=0)
    print(len(cases), "cases,", os.path.getsize(os.path.join(HERE, "family_ops.npz")), "bytes")


if __name__ == "__main__":
    main()
