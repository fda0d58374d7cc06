"""Max / Min / Pow and the one-line unary operators on the GPU against the oracle.

Exactly rounded expressions (max, min, neg, reciprocal, ceil, floor, sqrt, round, softsign, hard_swish) must give
identical codes.  The transcendental ones are evaluated in double by CUDA's libm here and by glibc's in the oracle,
both accurate to about one unit in the last place of a double: the gate is 2 units in the last place of the OUTPUT
type (in practice float32 and narrower outputs are identical) plus 2^-50 absolute, which covers the expressions that
add 1 to a libm result before using it (softplus, gelu: a last-place difference of the inner call becomes an absolute
2^-52 of the sum whatever the size of the final value)."""
import zlib

import numpy as np
import pytest

import gpu_ops as gpu
from datagen import FLOAT_DTYPES, assert_same_codes, from_f64, make, to_f64

pytestmark = pytest.mark.gpu

EXACT = ("neg", "reciprocal", "ceil", "floor", "sqrt", "round", "softsign", "hard_swish")
LIBM = ("exp", "log", "sigmoid", "tanh", "sin", "tan", "atan", "softplus", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "erf", "gelu")
ULP = {"float32": 2.0 ** -23, "float64": 2.0 ** -52, "float16": 2.0 ** -10, "bfloat16": 2.0 ** -7, "float8_e4m3": 2.0 ** -3}
PAIRS = (("float32", "float32"), ("float16", "float16"), ("bfloat16", "float32"), ("float64", "float64"), ("int8", "float32"),
         ("float32", "int32"), ("float8_e4m3", "float16"))


def _input(rng, x_dt):
    x = make(rng, (37, 129), x_dt, -3, 3) if x_dt in FLOAT_DTYPES else make(rng, (37, 129), x_dt)
    if x_dt == "float32":
        x.reshape(-1)[:8] = [0.0, -0.0, 1.0, -1.0, 0.5, np.inf, -np.inf, np.nan]
    return x


@pytest.mark.parametrize("op", EXACT)
def test_exactly_rounded_unary_operators(port, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for x_dt, out_dt in PAIRS:
        x = _input(rng, x_dt)
        assert_same_codes(gpu.unary_math(op, x, x_dt, out_dt), port.unary_math(op, x, x_dt, out_dt), out_dt, f"{op} {x_dt}->{out_dt}")


@pytest.mark.parametrize("op", LIBM)
def test_libm_unary_operators(port, op):
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for x_dt, out_dt in PAIRS:
        x = _input(rng, x_dt)
        got, want = gpu.unary_math(op, x, x_dt, out_dt), port.unary_math(op, x, x_dt, out_dt)
        if out_dt == "int32":
            assert np.abs(got.astype(np.int64) - want.astype(np.int64)).max() <= 1            # a value at a .5 tie may round either way
            continue
        g, w = to_f64(got, out_dt), to_f64(want, out_dt)
        with np.errstate(invalid="ignore"):
            ok = (np.isnan(g) & np.isnan(w)) | (g == w) | (np.abs(g - w) <= 2 * ULP[out_dt] * np.abs(w) + 2.0 ** -50)
        assert ok.all(), f"{op} {x_dt}->{out_dt}: {int((~ok).sum())} outside 2 ulp"
        if out_dt in ("float32", "float16"):
            assert np.mean((g == w) | (np.isnan(g) & np.isnan(w))) > 0.9999


@pytest.mark.parametrize("plan", [("float32", "float32", "float32"), ("float16", "float16", "float16"), ("bfloat16", "float32", "float32"),
                                  ("int8", "int8", "int8"), ("int32", "int32", "int32"), ("int32", "float16", "float64"), ("uint8", "int8", "int16"),
                                  ("int64", "int64", "int64"), ("float32", "float32", "int8")], ids="-".join)
@pytest.mark.parametrize("op", ["max", "min"])
def test_max_min_bit_exact_with_broadcasting(port, op, plan):
    a_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32((op + "-".join(plan)).encode()))
    for a_shape, b_shape in (((9, 31, 64), (9, 31, 64)), ((9, 31, 64), (31, 1)), ((9, 31, 64), (64,))):
        a, b = make(rng, a_shape, a_dt), make(rng, b_shape, b_dt)
        if a_dt == "float32":
            a.reshape(-1)[:6] = [np.nan, 1.0, np.inf, -np.inf, 0.0, -0.0]
            b.reshape(-1)[:6] = [1.0, np.nan, 1.0, 2.0, -0.0, 0.0]
        assert_same_codes(gpu.binary(op, a, a_dt, b, b_dt, out_dt), port.binary(op, a, a_dt, b, b_dt, out_dt), out_dt, f"{op} {plan}")


@pytest.mark.parametrize("plan", [("float32", "float32", "float32"), ("float16", "float16", "float16"), ("int8", "int8", "int8"),
                                  ("int32", "float32", "float32"), ("float64", "float64", "float64")], ids="-".join)
def test_pow_within_two_ulp(port, plan):
    a_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32(("pow" + "-".join(plan)).encode()))
    a = make(rng, (64, 200), a_dt, 0.1, 4) if a_dt in FLOAT_DTYPES else make(rng, (64, 200), a_dt, 1, 6)
    b = make(rng, (200,), b_dt, -3, 3) if b_dt in FLOAT_DTYPES else make(rng, (200,), b_dt, 0, 2)
    got, want = gpu.binary("pow", a, a_dt, b, b_dt, out_dt), port.binary("pow", a, a_dt, b, b_dt, out_dt)
    if out_dt == "int8":
        assert np.array_equal(got, want)
        return
    g, w = to_f64(got, out_dt), to_f64(want, out_dt)
    assert np.all((g == w) | (np.abs(g - w) <= 2 * ULP[out_dt] * np.abs(w)))
