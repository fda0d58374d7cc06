"""Generates tests/golden/adjacent_ops.npz + adjacent_ops.json from the reference's OWN C library
(oracle/_ref/tensor_ops_ref.so): Cast, Clip, AveragePool, GlobalAveragePool, BatchNormalization on small
seeded inputs.  Run where the reference sources are available:

    python tests/golden/make_adjacent_golden.py
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
from datagen import from_f64, make  # noqa: E402


def main():
    ref = oracle.HostOracle("ref")
    rng = np.random.default_rng(20240611)
    arrays, cases = {}, []

    def add(op, inputs, params, out):
        idx = len(cases)
        names = []
        for k, arr in enumerate(inputs):
            if arr is None:
                names.append(None)
            else:
                arrays[f"c{idx}_in{k}"] = np.ascontiguousarray(arr)
                names.append(f"c{idx}_in{k}")
        arrays[f"c{idx}_out"] = np.ascontiguousarray(out)
        cases.append({"id": idx, "op": op, "inputs": names, "params": params})

    edge = np.array([0.0, -0.0, 0.5, 1.5, 2.5, -2.5, 127.5, -128.5, 255.5, 448.0, 465.0, 61440.0, 65520.0, 2.0 ** -24, 1e-40, 3e38,
                     2147483648.0, -9.3e18, np.inf, -np.inf, np.nan])
    for x_dt, out_dt in (("float32", "int8"), ("float32", "int32"), ("float32", "float16"), ("float64", "int64"), ("float16", "uint8"),
                         ("bfloat16", "float32"), ("int32", "float16"), ("int8", "float8_e4m3"), ("float8_e5m2", "int16"), ("int64", "int64"),
                         ("float32", "float8_e5m2"), ("uint8", "bfloat16")):
        x = make(rng, (6, 9), x_dt)
        if x_dt in ("float32", "float64", "float16"):
            with np.errstate(all="ignore"):
                x.reshape(-1)[:edge.size] = from_f64(edge, x_dt)
        add("cast", [x], {"x_dt": x_dt, "out_dt": out_dt}, ref.cast(x, x_dt, out_dt))
    for x_dt, b_dt, out_dt in (("float32", "float32", "float32"), ("float16", "float32", "float16"), ("int8", "int8", "int8"), ("int32", "float32", "int32")):
        x = make(rng, (4, 5, 6), x_dt)
        lo, hi = from_f64(np.array([-3.0]), b_dt), from_f64(np.array([5.0]), b_dt)
        for lo_, hi_ in ((lo, hi), (lo, None), (None, hi)):
            add("clip", [x, lo_, hi_], {"x_dt": x_dt, "b_dt": b_dt, "out_dt": out_dt}, ref.clip(x, x_dt, lo_, b_dt, hi_, b_dt, out_dt))
    for x_dt, out_dt, xs, kernel, pads, strides, dil, inc in (
            ("float32", "float32", (2, 3, 9, 8), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1), 0),
            ("float32", "float32", (2, 3, 9, 8), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1), 1),
            ("float16", "float16", (1, 4, 12, 12), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1), 0),
            ("bfloat16", "float32", (1, 2, 10, 11), (3, 3), (2, 2, 2, 2), (1, 1), (2, 2), 1),
            ("int8", "int8", (2, 2, 7, 7), (3, 2), (1, 0, 1, 1), (1, 2), (1, 1), 0)):
        x = make(rng, xs, x_dt)
        add("average_pool", [x], {"x_dt": x_dt, "out_dt": out_dt, "kernel": kernel, "pads": pads, "strides": strides, "dilations": dil,
                                  "count_include_pad": inc}, ref.average_pool(x, x_dt, out_dt, kernel, pads, strides, dil, inc))
    for x_dt, out_dt, xs in (("float32", "float32", (4, 6, 7, 7)), ("float16", "float16", (2, 3, 5, 9)), ("int8", "float32", (1, 8, 4, 4))):
        x = make(rng, xs, x_dt)
        add("global_average_pool", [x], {"x_dt": x_dt, "out_dt": out_dt}, ref.global_average_pool(x, x_dt, out_dt))
    for x_dt, p_dt, out_dt, xs in (("float32", "float32", "float32", (3, 5, 6, 7)), ("float16", "float32", "float16", (2, 4, 5, 5)),
                                   ("float32", "float32", "float32", (4, 6)), ("float64", "float64", "float64", (2, 2, 3, 3))):
        x = make(rng, xs, x_dt)
        c = xs[1]
        scale, bias, mean = (from_f64(rng.normal(0, 1, c), p_dt) for _ in range(3))
        var = from_f64(rng.uniform(0.1, 2.0, c), p_dt)
        add("batch_norm", [x, scale, bias, mean, var], {"x_dt": x_dt, "p_dt": p_dt, "out_dt": out_dt, "epsilon": 1e-5},
            ref.batch_norm(x, x_dt, scale, bias, mean, var, p_dt, out_dt, 1e-5))
    np.savez_compressed(os.path.join(HERE, "adjacent_ops.npz"), **arrays)
    with open(os.path.join(HERE, "adjacent_ops.json"), "w") as f:
        json.dump(cases, f, indent=0)
    print(len(cases), "cases,", os.path.getsize(os.path.join(HERE, "adjacent_ops.npz")), "bytes")


if __name__ == "__main__":
    main()
