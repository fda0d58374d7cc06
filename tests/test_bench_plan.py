"""The benchmark's bookkeeping, checked without a GPU: the sweep has the launches the benchmark
configuration lists, and the algorithmic bytes per element are size(A) + size(out), plus size(B)
only when B has the full shape."""
import importlib.util
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
spec = importlib.util.spec_from_file_location("bench_module", os.path.join(ROOT, "bench.py"))
bench = importlib.util.module_from_spec(spec)
spec.loader.exec_module(bench)


def test_sweep_has_the_configured_launches():
    plan = bench.sweep_plan(64)
    assert len(plan) == 4 * 3 * 7 + 2 * 5 + 1 == 95
    assert sum(p["kind"] == "binary" for p in plan) == 84
    assert {p["op"] for p in plan} == {"add", "sub", "mul", "div", "relu", "abs", "cos"}
    assert ("int32", "float16", "float64") in {(p["a"], p["b"], p["o"]) for p in plan if p["kind"] == "binary"}


def test_algorithmic_bytes_per_element():
    n = 64 * 512 * 1024
    per_elem = {}
    for p in bench.sweep_plan(64):
        if p["kind"] == "binary":
            per_elem[(p["a"], p["b"], p["o"], p["bname"])] = p["bytes"] / n
    # broadcast B: its own bytes are negligible (2 KB / 4 KB); full B counts
    assert round(per_elem[("float32", "float32", "float32", "row")], 3) == 8 and per_elem[("float32", "float32", "float32", "full")] == 12
    assert round(per_elem[("float16", "float16", "float16", "vec")], 3) == 4 and per_elem[("bfloat16", "bfloat16", "bfloat16", "full")] == 6
    assert round(per_elem[("int8", "int8", "int8", "row")], 3) == 2 and per_elem[("int8", "int8", "int8", "full")] == 3
    assert round(per_elem[("int8", "float32", "float32", "row")], 3) == 5 and per_elem[("int8", "float32", "float32", "full")] == 9
    assert round(per_elem[("int32", "float16", "float64", "row")], 3) == 12 and per_elem[("int32", "float16", "float64", "full")] == 14
    unary = {p["label"]: p["bytes"] / n for p in bench.sweep_plan(64) if p["kind"] == "unary"}
    assert unary["relu float32"] == 8 and unary["abs int8"] == 2 and unary["cos float32"] == 8


def test_inputs_are_seeded_and_divisors_stay_away_from_zero():
    a1, c1, b1 = bench.host_inputs(1, seed=0)
    a2, c2, b2 = bench.host_inputs(1, seed=0)
    assert all(np.array_equal(a1[k], a2[k]) for k in a1) and np.array_equal(c1, c2)
    assert np.abs(c1).max() <= 10
    for (bname, dt, divisor), arr in b1.items():
        if divisor and dt == "float32":
            assert np.abs(arr).min() >= 0.5
        if divisor and dt in ("int32", "int8"):
            assert np.all(arr != 0)
