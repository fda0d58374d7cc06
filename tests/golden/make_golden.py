"""Generates tests/golden/hot_path.npz + hot_path.json from the reference's OWN C library.

Run where the reference sources are available (they are compiled, unchanged, by oracle/Makefile into
oracle/_ref/tensor_ops_ref.so):

    python tests/golden/make_golden.py

The reference project stores no golden vectors of its own (its harness draws unseeded random data),
so these fixtures are what pins the oracle and the CUDA library on machines where the reference
cannot be built.  Inputs are seeded; every array is small (the whole file is well under 1 MB).
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
from datagen import make, from_f64  # noqa: E402


def main():
    ref = oracle.HostOracle("ref")
    rng = np.random.default_rng(20240607)
    arrays, cases = {}, []

    def add(op, inputs, params, out):
        idx = len(cases)
        names = []
        for k, arr in enumerate(inputs):
            key = f"c{idx}_in{k}"
            if arr is None:
                names.append(None)
            else:
                arrays[key] = np.ascontiguousarray(arr)
                names.append(key)
        arrays[f"c{idx}_out"] = np.ascontiguousarray(out)
        cases.append({"id": idx, "op": op, "inputs": names, "params": params})

    edge = np.array([0.0, -0.0, 0.5, 1.5, 2.5, -2.5, 127.5, -128.5, 448.0, 464.0, 465.0, 57344.0, 61440.0, 65504.0, 65520.0,
                     2.0 ** -6 * 0.999, 2.0 ** -14 * 0.999, 2.0 ** -24, 2.0 ** -24 * 0.99, 2.0 ** -25, 1e-40, 3e38, np.inf, -np.inf, np.nan])
    # unary
    for op in ("relu", "abs"):
        for x_dt, out_dt in (("float32", "float32"), ("float16", "float16"), ("bfloat16", "bfloat16"), ("int8", "int8"),
                             ("int32", "int32"), ("float8_e4m3", "float8_e4m3"), ("float8_e5m2", "float16"), ("float32", "int8"),
                             ("float32", "float8_e4m3"), ("float32", "float8_e5m2"), ("float32", "float16"), ("int4", "int4"),
                             ("float64", "bfloat16"), ("int64", "int16"), ("uint8", "float32")):
            x = make(rng, (8, 16), x_dt)
            if x_dt in ("float32", "float64"):
                with np.errstate(all="ignore"):
                    x.reshape(-1)[:edge.size] = from_f64(edge, x_dt)
            add(op, [x], {"x_dt": x_dt, "out_dt": out_dt}, ref.unary(op, x, x_dt, out_dt))
    for x_dt, out_dt in (("float32", "float32"), ("float16", "float16"), ("bfloat16", "float32"), ("float64", "float64"), ("int8", "float32")):
        vals = np.concatenate([rng.uniform(-10, 10, 200), rng.uniform(-1e4, 1e4, 50), [0.0, 6.283185307179586, 12.566370614359172, 1e-30]])
        x = from_f64(np.clip(vals, -120, 120) if x_dt == "int8" else vals, x_dt)
        add("cos", [x], {"x_dt": x_dt, "out_dt": out_dt}, ref.unary("cos", x, x_dt, out_dt))
    # binary (same shape and broadcast)
    plans = [("float32", "float32", "float32"), ("float16", "float16", "float16"), ("bfloat16", "bfloat16", "bfloat16"),
             ("int32", "int32", "int32"), ("int8", "int8", "int8"), ("int8", "float32", "float32"), ("int32", "float16", "float64"),
             ("uint8", "int8", "int16"), ("float8_e4m3", "float8_e4m3", "float8_e4m3"), ("float32", "float32", "int8"),
             ("int64", "float32", "float64"), ("float16", "float32", "float16")]
    for op in ("add", "sub", "mul", "div"):
        for a_dt, b_dt, o_dt in plans:
            a = make(rng, (6, 4, 8), a_dt)
            b = make(rng, (1, 4, 1), b_dt)
            if b_dt.startswith("int") or b_dt == "uint8":
                b.reshape(-1)[0] = 0
            add(op, [a, b], {"a_dt": a_dt, "b_dt": b_dt, "out_dt": o_dt}, ref.binary(op, a, a_dt, b, b_dt, o_dt))
    sat_a = np.array([127, -128, 100, -100, 127, -128, 0, 1], dtype=np.int8)
    sat_b = np.array([127, -128, 100, 100, -1, -1, 0, 0], dtype=np.int8)
    for op in ("add", "sub", "mul", "div"):
        add(op, [sat_a, sat_b], {"a_dt": "int8", "b_dt": "int8", "out_dt": "int8"}, ref.binary(op, sat_a, "int8", sat_b, "int8", "int8"))
    # quantize / dequantize
    xq = np.concatenate([rng.standard_normal(480), [0.49, 0.5, 0.51, 1.5, 2.5, -0.5, 17.3, 1e9, -1e9, np.inf, -np.inf, np.nan, 0.01, 0.03, -0.05, 28.0]])
    xq = xq.astype(np.float32).reshape(2, 8, 31)
    for out_dt, z_dt, zp, s in (("int8", "int8", 0, 0.02), ("uint8", "uint8", 128, 0.02), ("float8_e4m3", "int8", 0, 1 / 16),
                                ("float8_e5m2", "int8", 0, 1 / 16), ("int8", "int8", 3, 0.0), ("int32", "int32", 5, 3.0)):
        sv = np.array([s], np.float32)
        zv = np.array([zp]).astype(np.uint8 if z_dt == "uint8" else (np.int32 if z_dt == "int32" else np.int8))
        add("quantize", [xq, sv, zv], {"x_dt": "float32", "s_dt": "float32", "z_dt": z_dt, "out_dt": out_dt, "axis": None},
            ref.quantize(xq, "float32", sv, "float32", zv, z_dt, out_dt))
    s_ax = rng.uniform(0.01, 0.05, 8).astype(np.float32)
    z_ax = rng.integers(-8, 9, 8).astype(np.int8)
    add("quantize", [xq, s_ax, z_ax], {"x_dt": "float32", "s_dt": "float32", "z_dt": "int8", "out_dt": "int8", "axis": 1},
        ref.quantize(xq, "float32", s_ax, "float32", z_ax, "int8", "int8", axis=1))
    for x_dt in ("int8", "uint8", "float8_e4m3", "float8_e5m2", "int32"):
        xd = make(rng, (2, 8, 31), x_dt)
        zd = make(rng, (1,), x_dt) if not x_dt.startswith("float8") else np.array([0], np.uint8)
        sd = rng.uniform(0.005, 0.02, (1, 8, 1)).astype(np.float32)
        for out_dt in ("float32", "bfloat16"):
            add("dequantize", [xd, sd, zd], {"x_dt": x_dt, "s_dt": "float32", "z_dt": x_dt, "out_dt": out_dt},
                ref.dequantize(xd, x_dt, sd, "float32", zd, x_dt, out_dt))
    # conv / pool / gemm / softmax
    for x_dt, w_dt, b_dt, o_dt, xs, ws, pads, st, dil, g in (
            ("float32", "float32", "float32", "float32", (2, 4, 9, 8), (6, 2, 3, 2), (2, 1, 0, 1), (2, 1), (2, 2), 2),
            ("bfloat16", "bfloat16", "bfloat16", "bfloat16", (1, 8, 6, 6), (8, 1, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 8),
            ("float8_e4m3", "float8_e4m3", None, "float16", (2, 3, 9, 9), (4, 3, 3, 3), (0, 0, 0, 0), (2, 2), (1, 1), 1),
            ("float16", "float16", "float32", "float16", (1, 2, 8, 8), (4, 2, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 1)):
        x = make(rng, xs, x_dt, -2, 2)
        w = make(rng, ws, w_dt, -1, 1)
        b = None if b_dt is None else make(rng, (ws[0],), b_dt, -1, 1)
        add("conv2d", [x, w, b], {"x_dt": x_dt, "w_dt": w_dt, "b_dt": b_dt or "float32", "out_dt": o_dt, "pads": pads, "strides": st,
                                  "dilations": dil, "group": g},
            ref.conv2d(x, x_dt, w, w_dt, b, b_dt or "float32", o_dt, pads, st, dil, g))
    for x_dt, o_dt, xs, k, pads, st, dil in (("float32", "float32", (2, 3, 9, 8), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
                                             ("bfloat16", "bfloat16", (1, 2, 8, 8), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
                                             ("float16", "float32", (1, 2, 12, 12), (3, 2), (2, 0, 1, 1), (1, 2), (2, 2)),
                                             ("float32", "float32", (1, 1, 3, 3), (2, 2), (2, 2, 2, 2), (3, 3), (1, 1))):
        x = make(rng, xs, x_dt)
        if x_dt == "float32":
            x.reshape(-1)[::7] = np.nan
        add("max_pool", [x], {"x_dt": x_dt, "out_dt": o_dt, "kernel": k, "pads": pads, "strides": st, "dilations": dil},
            ref.max_pool(x, x_dt, o_dt, k, pads, st, dil))
    for a_dt, b_dt, c_dt, o_dt, ash, bsh, csh, al, be, ta, tb in (
            ("float32", "float32", "float32", "float32", (2, 3), (3, 4), (4,), 1.0, 1.0, 0, 0),
            ("float8_e5m2", "float8_e4m3", "float16", "bfloat16", (8, 16), (12, 16), (12,), 0.5, 1.0, 0, 1),
            ("float32", "float32", "float32", "float32", (7, 5), (7, 9), (5, 1), 1.25, -0.5, 1, 0),
            ("bfloat16", "bfloat16", "float32", "bfloat16", (6, 10), (4, 10), (6, 4), 1.0, 2.0, 0, 1),
            ("float16", "float16", None, "float32", (16, 32), (32, 8), None, 1.0, 1.0, 0, 0)):
        a = make(rng, ash, a_dt, -2, 2)
        b = make(rng, bsh, b_dt, -2, 2)
        c = None if c_dt is None else make(rng, csh, c_dt, -1, 1)
        add("gemm", [a, b, c], {"a_dt": a_dt, "b_dt": b_dt, "c_dt": c_dt or "float32", "out_dt": o_dt, "alpha": al, "beta": be,
                                "transA": ta, "transB": tb},
            ref.gemm(a, a_dt, b, b_dt, c, c_dt or "float32", o_dt, al, be, ta, tb))
    for x_dt, o_dt, shape, axis in (("float32", "float32", (2, 5), -1), ("float16", "float16", (4, 64), 1),
                                    ("float32", "float32", (3, 7, 5), 1), ("bfloat16", "float32", (3, 100), -1)):
        x = make(rng, shape, x_dt)
        add("softmax", [x], {"x_dt": x_dt, "out_dt": o_dt, "axis": axis}, ref.softmax(x, x_dt, o_dt, axis))

    np.savez_compressed(os.path.join(HERE, "hot_path.npz"), **arrays)
    with open(os.path.join(HERE, "hot_path.json"), "w") as f:
        json.dump({"generator": "tests/golden/make_golden.py", "source": "tensor_ops/tensor_ops.c compiled unchanged (gcc -O3 -fopenmp)",
                   "cases": cases}, f, indent=0)
    print(f"{len(cases)} cases, {sum(a.nbytes for a in arrays.values())} bytes of arrays")


if __name__ == "__main__":
    main()
