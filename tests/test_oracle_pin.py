"""Pins the C restatement (oracle/oracle.c) to the reference's own compiled tensor_ops.c.

Every case runs both libraries on the same seeded inputs and demands identical output codes
(any NaN equals any NaN).  The plans mirror the reference harness (numerical_correctness.py:432-567)
and add what it leaves untested: uint8 / fp8 quantisation, per-axis scales, pooling with padding
and dilation, dilated and grouped convolution, every Gemm bias shape.
Skipped when no compiled reference is present (the golden-vector tests then carry the pin).
"""
import zlib

import numpy as np
import pytest

from datagen import ALL_DTYPES, FLOAT_DTYPES, INT_DTYPES, assert_same_codes, from_f64, make, to_f64

OUT_SAMPLE = ("float8_e4m3", "float8_e5m2", "float16", "bfloat16", "float32", "float64",
              "int4", "int8", "uint8", "int16", "int32", "int64")


def _special_values(dtype):
    """Hand-picked edge inputs for a dtype, as float64 before encoding."""
    v = [0.0, -0.0, 1.0, -1.0, 0.5, 1.5, 2.5, -2.5, 127.4, 127.5, 128.5, -128.5, 255.5, 447.0, 448.0,
         449.0, 464.0, 465.0, 480.0, 57344.0, 61439.0, 61440.0, 65504.0, 65519.0, 65520.0, 1e5, -1e5,
         2.0 ** -6, 2.0 ** -6 * 0.999, 2.0 ** -7, 2.0 ** -9, 2.0 ** -14, 2.0 ** -14 * 0.999, 2.0 ** -15,
         2.0 ** -24, 2.0 ** -24 * 0.99, 2.0 ** -25, 2.0 ** -24 * 1.5, 6.1e-5, 5.9e-8, 3e38, -3e38,
         2147483647.0, 2147483648.0, -2147483649.0, 9.3e18, -9.3e18, 1e-40, np.inf, -np.inf, np.nan]
    return np.array(v, dtype=np.float64)


@pytest.mark.parametrize("x_dt", ALL_DTYPES)
@pytest.mark.parametrize("op", ["relu", "abs"])
def test_unary_all_dtype_pairs(port, ref, op, x_dt):
    rng = np.random.default_rng(zlib.crc32(f"{op}{x_dt}".encode()))
    x = make(rng, (37, 29), x_dt)
    if x_dt in FLOAT_DTYPES and x_dt not in ("float8_e4m3", "float8_e5m2"):
        with np.errstate(over="ignore", invalid="ignore"):
            x.reshape(-1)[:51] = from_f64(_special_values(x_dt), x_dt)
    for out_dt in OUT_SAMPLE:
        assert_same_codes(port.unary(op, x, x_dt, out_dt), ref.unary(op, x, x_dt, out_dt), out_dt,
                          f"{op} {x_dt}->{out_dt}")


@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64", "int8", "int32", "float8_e5m2"])
def test_cos(port, ref, x_dt):
    rng = np.random.default_rng(7)
    if x_dt == "float8_e5m2":                 # finite codes only: NaN/Inf inputs are undefined upstream
        x = rng.integers(0, 0x7C, size=4096, dtype=np.uint8) | (rng.integers(0, 2, size=4096, dtype=np.uint8) << 7)
    else:
        x = np.concatenate([rng.uniform(-10, 10, 20000), rng.uniform(-1e4, 1e4, 20000),
                            [0.0, -0.0, 2 * np.pi, 4 * np.pi, 6.283185307179586, 6.2831854820251465,
                             12.566370614359172, 1e30, -1e30, 1e-30]])
        if x_dt == "float16":                 # stay finite: Inf indexes outside the table upstream
            x = np.clip(x, -60000, 60000)
        x = from_f64(x if x_dt not in INT_DTYPES else np.clip(x, -120, 120), x_dt)
    for out_dt in ("float32", "float16", "bfloat16", "float64", "int8"):
        assert_same_codes(port.unary("cos", x, x_dt, out_dt), ref.unary("cos", x, x_dt, out_dt), out_dt,
                          f"cos {x_dt}->{out_dt}")


def test_cos_table_matches_reference_lookup(port, ref):
    """Probing the reference at the exact table knots returns the table itself."""
    table = port.cos_table()
    knots = np.arange(4097, dtype=np.float64) * (2.0 * np.pi) / 4096.0
    got = ref.unary("cos", knots[:4096], "float64", "float64")
    # fmod/scale round-off moves a probe off its knot by at most a few 1e-13 of a cell
    assert np.max(np.abs(got - table[:4096])) < 1e-12


BINARY_PLANS = [  # (a_dt, b_dt, out_dt) -- numerical_correctness.py:433-470 plus BASELINE config 2
    ("float32", "float32", "float32"), ("float16", "float16", "float16"), ("bfloat16", "bfloat16", "bfloat16"),
    ("float64", "float64", "float64"), ("int32", "int32", "int32"), ("int8", "int8", "int8"),
    ("int8", "float32", "float32"), ("int32", "float16", "float64"), ("int4", "int4", "int4"),
    ("uint8", "int8", "int16"), ("int64", "float32", "float64"), ("bfloat16", "float32", "float32"),
    ("bfloat16", "float16", "float32"), ("float8_e4m3", "float8_e4m3", "float8_e4m3"),
    ("float8_e5m2", "float8_e4m3", "float16"), ("float8_e5m2", "float8_e5m2", "float8_e5m2"),
    ("float16", "float32", "float16"), ("float32", "float32", "int8"), ("float32", "int8", "int32"),
    ("float16", "float16", "int4"), ("int16", "int16", "int16"), ("int64", "int64", "int64"),
    ("uint8", "uint8", "uint8"), ("int32", "int32", "float32"), ("float64", "float32", "float32"),
    ("int8", "int8", "int32"), ("float32", "float32", "float8_e4m3"), ("int64", "int32", "bfloat16"),
]


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("plan", BINARY_PLANS, ids=lambda p: "-".join(p))
def test_binary(port, ref, op, plan):
    a_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32(repr((op,) + plan).encode()))
    a = make(rng, (64, 64), a_dt)
    b = make(rng, (64, 64), b_dt)
    if b_dt in INT_DTYPES:
        b.reshape(-1)[::97] = 0               # integer division by zero is defined (saturates)
    assert_same_codes(port.binary(op, a, a_dt, b, b_dt, out_dt), ref.binary(op, a, a_dt, b, b_dt, out_dt),
                      out_dt, f"{op} {plan}")


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_saturation_and_wrap(port, ref, op):
    """Values at the integer limits: saturating stores, int64 wrap, x86 float->int conversion."""
    a = np.array([127, -128, 100, -100, 127, -128, 0, 1], dtype=np.int8)
    b = np.array([127, -128, 100, 100, -1, -1, 0, 0], dtype=np.int8)
    assert_same_codes(port.binary(op, a, "int8", b, "int8", "int8"), ref.binary(op, a, "int8", b, "int8", "int8"), "int8")
    a32 = np.array([2 ** 31 - 1, -2 ** 31, 2 ** 31 - 1, 65536, -2 ** 31, 7, -7, 0], dtype=np.int32)
    b32 = np.array([2 ** 31 - 1, -2 ** 31, -2 ** 31, 65536, -1, 0, 0, 0], dtype=np.int32)
    for out in ("int32", "int64", "int16", "uint8"):
        assert_same_codes(port.binary(op, a32, "int32", b32, "int32", out), ref.binary(op, a32, "int32", b32, "int32", out), out)
    a64 = np.array([2 ** 62, -2 ** 62, 2 ** 63 - 1, 3, 2 ** 40], dtype=np.int64)
    b64 = np.array([2 ** 62, -2 ** 62, 2, 0, 2 ** 40], dtype=np.int64)
    assert_same_codes(port.binary(op, a64, "int64", b64, "int64", "int64"), ref.binary(op, a64, "int64", b64, "int64", "int64"), "int64")
    af = np.array([np.nan, np.inf, -np.inf, 1e30, -1e30, 2.5, 3.5, -2.5, 0.5, 1e10], dtype=np.float32)
    bf = np.array([1, 1, 1, 1, 1, 1, 1, 1, 1, 1], dtype=np.float32)
    for out in ("int8", "uint8", "int32", "int64", "int4"):
        assert_same_codes(port.binary(op, af, "float32", bf, "float32", out), ref.binary(op, af, "float32", bf, "float32", out), out)


@pytest.mark.parametrize("out_dt", ["int8", "uint8", "int4", "int16", "int32", "float8_e4m3", "float8_e5m2", "float16", "float32"])
@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64"])
def test_quantize(port, ref, x_dt, out_dt):
    rng = np.random.default_rng(11)
    x = make(rng, (2, 16, 12, 12), x_dt)
    zp_dt = out_dt if out_dt in INT_DTYPES else "int8"
    # per tensor
    s = np.array([0.02], dtype=np.float32)
    z = np.array([3], dtype=np.int64).astype(np.int8 if zp_dt != "uint8" else np.uint8)
    assert_same_codes(port.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt),
                      ref.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt), out_dt, "per-tensor")
    # per axis (axis 1), including a zero scale
    s = rng.uniform(0.01, 0.05, 16).astype(np.float32)
    s[5] = 0.0
    z = rng.integers(0, 9, 16).astype(z.dtype)
    assert_same_codes(port.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt, axis=1),
                      ref.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt, axis=1), out_dt, "per-axis")


def test_quantize_edge_values(port, ref):
    x = np.array([0.49, 0.5, 0.51, 1.5, 2.5, -0.5, -1.5, 17.3, 1e9, -1e9, np.inf, -np.inf, np.nan,
                  2.55, 2.56, -2.57, 448 / 16, 449, 1e-9, 60000.0, 70000.0], dtype=np.float32)
    for out_dt, zp_dt, zp in (("int8", "int8", 0), ("uint8", "uint8", 128), ("float8_e4m3", "int8", 0),
                              ("float8_e5m2", "int8", 0), ("int32", "int32", 5)):
        for s in (1.0, 0.02, 1 / 16, 3.0):
            sv = np.array([s], dtype=np.float32)
            zv = np.array([zp]).astype(np.uint8 if zp_dt == "uint8" else np.int32)
            assert_same_codes(port.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt),
                              ref.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt), out_dt, f"{out_dt} s={s}")


@pytest.mark.parametrize("x_dt", ["int8", "uint8", "int32", "float8_e4m3", "float8_e5m2", "int4", "int16"])
@pytest.mark.parametrize("out_dt", ["float32", "float16", "bfloat16", "float64"])
def test_dequantize(port, ref, x_dt, out_dt):
    rng = np.random.default_rng(13)
    x = make(rng, (3, 8, 10, 10), x_dt)
    zp_dt = x_dt
    z = make(rng, (1,), zp_dt) if x_dt not in ("float8_e4m3", "float8_e5m2") else np.array([0], dtype=np.uint8)
    s = np.array([0.0173], dtype=np.float32)
    assert_same_codes(port.dequantize(x, x_dt, s, "float32", z, zp_dt, out_dt),
                      ref.dequantize(x, x_dt, s, "float32", z, zp_dt, out_dt), out_dt)
    s = rng.uniform(0.005, 0.02, (1, 8, 1, 1)).astype(np.float32)
    z = np.broadcast_to(z, (1, 8, 1, 1)).copy()
    assert_same_codes(port.dequantize(x, x_dt, s, "float32", z, zp_dt, out_dt),
                      ref.dequantize(x, x_dt, s, "float32", z, zp_dt, out_dt), out_dt)


CONV_PLANS = [  # x_dt, w_dt, b_dt, out_dt, xshape, wshape, pads, strides, dilations, group
    ("float32", "float32", None, "float32", (1, 1, 5, 5), (1, 1, 3, 3), (0, 0, 0, 0), (1, 1), (1, 1), 1),
    ("float16", "float16", "float32", "float16", (1, 2, 8, 8), (4, 2, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 1),
    ("float8_e4m3", "float8_e4m3", None, "float16", (2, 3, 9, 9), (4, 3, 3, 3), (0, 0, 0, 0), (2, 2), (1, 1), 1),
    ("bfloat16", "bfloat16", "bfloat16", "bfloat16", (1, 8, 6, 6), (8, 1, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 8),
    ("float32", "float32", "float32", "float32", (2, 4, 11, 10), (6, 2, 3, 2), (2, 1, 0, 1), (2, 1), (2, 2), 2),
    ("int8", "int8", "int32", "int32", (1, 3, 7, 7), (5, 3, 3, 3), (1, 1, 1, 1), (1, 1), (1, 1), 1),
    ("float32", "int8", "float32", "float32", (1, 3, 7, 7), (5, 3, 1, 1), (0, 0, 0, 0), (1, 1), (1, 1), 1),
    ("float64", "float64", None, "float64", (1, 2, 6, 6), (2, 2, 5, 5), (2, 2, 2, 2), (1, 1), (1, 1), 1),
]


@pytest.mark.parametrize("plan", CONV_PLANS, ids=lambda p: f"{p[0]}-{p[3]}-g{p[9]}")
def test_conv2d(port, ref, plan):
    x_dt, w_dt, b_dt, out_dt, xs, ws, pads, strides, dil, group = plan
    rng = np.random.default_rng(17)
    x = make(rng, xs, x_dt, -2, 2) if x_dt not in INT_DTYPES else make(rng, xs, x_dt)
    w = make(rng, ws, w_dt, -1, 1) if w_dt not in INT_DTYPES else make(rng, ws, w_dt)
    b = None if b_dt is None else make(rng, (ws[0],), b_dt)
    args = (x, x_dt, w, w_dt, b, b_dt or "float32", out_dt, pads, strides, dil, group)
    assert_same_codes(port.conv2d(*args), ref.conv2d(*args), out_dt)


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (1, 1, 4, 4), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("bfloat16", "bfloat16", (2, 3, 16, 16), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("float32", "float32", (2, 4, 15, 14), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float16", "float32", (1, 2, 12, 12), (3, 2), (2, 0, 1, 1), (1, 2), (2, 2)),
    ("int8", "int8", (1, 2, 9, 9), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float8_e4m3", "float8_e4m3", (1, 2, 9, 9), (2, 2), (0, 0, 0, 0), (1, 1), (1, 1)),
    ("float32", "float32", (1, 1, 3, 3), (2, 2), (2, 2, 2, 2), (3, 3), (1, 1)),   # windows made only of padding
], ids=lambda p: f"{p[0]}-{p[2]}-k{p[3]}")
def test_max_pool(port, ref, plan):
    x_dt, out_dt, xs, kernel, pads, strides, dil = plan
    rng = np.random.default_rng(19)
    x = make(rng, xs, x_dt)
    if x_dt == "float32":
        x.reshape(-1)[::7] = np.nan
        x.reshape(-1)[3::11] = -np.inf
    args = (x, x_dt, out_dt, kernel, pads, strides, dil)
    assert_same_codes(port.max_pool(*args), ref.max_pool(*args), out_dt)


GEMM_PLANS = [  # a_dt, b_dt, c_dt, out_dt, ashape, bshape, cshape, alpha, beta, tA, tB
    ("float32", "float32", "float32", "float32", (2, 3), (3, 4), (4,), 1.0, 1.0, 0, 0),
    ("float16", "float16", None, "float32", (16, 32), (32, 8), None, 1.0, 1.0, 0, 0),
    ("float8_e5m2", "float8_e4m3", "float16", "bfloat16", (8, 16), (12, 16), (12,), 0.5, 1.0, 0, 1),
    ("float32", "float32", "float32", "float32", (7, 5), (7, 9), (5, 1), 1.25, -0.5, 1, 0),
    ("bfloat16", "bfloat16", "float32", "bfloat16", (6, 10), (4, 10), (6, 4), 1.0, 2.0, 0, 1),
    ("float32", "float32", "float32", "float32", (10, 6), (4, 10), (1,), 1.0, 1.0, 1, 1),
    ("int8", "int8", "int32", "int32", (5, 7), (7, 3), (1, 3), 1.0, 1.0, 0, 0),
    ("float32", "float32", "float32", "float32", (5, 5), (5, 5), (5,), 1.0, 1.0, 0, 0),  # M == N: 1-D C goes per column
    ("float64", "float64", "float64", "float64", (4, 6), (6, 4), (4, 1), 1.0, 1.0, 0, 0),
]


@pytest.mark.parametrize("plan", GEMM_PLANS, ids=lambda p: f"{p[0]}-{p[3]}-{p[9]}{p[10]}")
def test_gemm(port, ref, plan):
    a_dt, b_dt, c_dt, out_dt, ash, bsh, csh, alpha, beta, ta, tb = plan
    rng = np.random.default_rng(23)
    a = make(rng, ash, a_dt, -2, 2) if a_dt not in INT_DTYPES else make(rng, ash, a_dt)
    b = make(rng, bsh, b_dt, -2, 2) if b_dt not in INT_DTYPES else make(rng, bsh, b_dt)
    c = None if c_dt is None else make(rng, csh, c_dt)
    args = (a, a_dt, b, b_dt, c, c_dt or "float32", out_dt, alpha, beta, ta, tb)
    assert_same_codes(port.gemm(*args), ref.gemm(*args), out_dt)


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (2, 5), -1), ("float16", "float16", (4, 64), 1), ("float8_e4m3", "float8_e4m3", (2, 10), 1),
    ("float32", "float32", (3, 7, 5), 1), ("float32", "float32", (3, 7, 5), 0), ("bfloat16", "float32", (6, 1000), -1),
    ("float64", "float64", (5, 33), 1), ("float32", "float16", (2, 3, 4, 5), 2),
], ids=lambda p: f"{p[0]}-{p[2]}-ax{p[3]}")
def test_softmax(port, ref, plan):
    x_dt, out_dt, shape, axis = plan
    rng = np.random.default_rng(29)
    if x_dt == "float8_e4m3":                 # keep NaN codes out: NaN rows are compared separately
        x = rng.integers(0, 0x7F, size=shape, dtype=np.uint8) | (rng.integers(0, 2, size=shape, dtype=np.uint8) << 7)
    else:
        x = make(rng, shape, x_dt)
    assert_same_codes(port.softmax(x, x_dt, out_dt, axis), ref.softmax(x, x_dt, out_dt, axis), out_dt)


def test_flatten(port, ref):
    rng = np.random.default_rng(31)
    for dt in ("float32", "int8", "bfloat16", "float64"):
        x = make(rng, (2, 3, 4, 5), dt)
        assert_same_codes(port.flatten(x, dt, (2, 60)), ref.flatten(x, dt, (2, 60)), dt)


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float8_e4m3", "float8_e5m2"])
def test_codec_exhaustive_against_reference(port, ref, dt):
    """Encode: a dense sweep of float32 inputs through Relu-free identity (Add with zero).
    Decode: every code of the format."""
    nbits = 16 if dt in ("float16", "bfloat16") else 8
    codes = np.arange(2 ** nbits, dtype=np.uint32).astype(np.uint16 if nbits == 16 else np.uint8)
    if dt == "float16":
        codes = codes.view(np.float16)
    zero = np.zeros(codes.shape, dtype=np.float32)
    # decode every code to float32 (x + 0.0 in double is exact, -0 + 0 = +0 in both libraries)
    assert_same_codes(port.binary("add", codes, dt, zero, "float32", "float32"),
                      ref.binary("add", codes, dt, zero, "float32", "float32"), "float32", "decode")
    # encode: all float32 values whose low 12 bits are one of a few patterns (2^20 * 6 inputs)
    hi = np.arange(2 ** 20, dtype=np.uint32) << 12
    for low in (0x000, 0x001, 0x7FF, 0x800, 0x801, 0xFFF):
        x = (hi | np.uint32(low)).view(np.float32)
        assert_same_codes(port.unary("abs", x, "float32", dt), ref.unary("abs", x, "float32", dt), dt, f"encode low={low:#x}")


# ---- operators around the hot path: Cast, Clip, AveragePool, GlobalAveragePool, BatchNormalization --------------------
@pytest.mark.parametrize("x_dt", ALL_DTYPES)
def test_cast_all_dtype_pairs(port, ref, x_dt):
    """float32 / float64 / float16 / bfloat16 -> integer truncates; everything else takes the generic store."""
    rng = np.random.default_rng(zlib.crc32(f"cast{x_dt}".encode()))
    x = make(rng, (33, 21), x_dt)
    if x_dt in FLOAT_DTYPES and x_dt not in ("float8_e4m3", "float8_e5m2"):
        with np.errstate(over="ignore", invalid="ignore"):
            x.reshape(-1)[:51] = from_f64(_special_values(x_dt), x_dt)
    for out_dt in OUT_SAMPLE:
        assert_same_codes(port.cast(x, x_dt, out_dt), ref.cast(x, x_dt, out_dt), out_dt, f"cast {x_dt}->{out_dt}")


@pytest.mark.parametrize("plan", [("float32", "float32", "float32"), ("float16", "float32", "float16"), ("int8", "int8", "int8"),
                                  ("int32", "float32", "int32"), ("bfloat16", "bfloat16", "float32"), ("float64", "float64", "float64"),
                                  ("float8_e4m3", "float32", "float8_e4m3"), ("uint8", "uint8", "int16")], ids="-".join)
def test_clip(port, ref, plan):
    x_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32("clip".encode() + "-".join(plan).encode()))
    x = make(rng, (6, 5, 7), x_dt)
    if x_dt in ("float32", "float64"):
        x.reshape(-1)[:4] = [np.nan, np.inf, -np.inf, -0.0]
    lo = from_f64(np.array([-3.0]), b_dt) if b_dt not in ("uint8",) else np.array([2], np.uint8)
    hi = from_f64(np.array([5.0]), b_dt) if b_dt not in ("uint8",) else np.array([9], np.uint8)
    for lo_, hi_ in ((lo, hi), (lo, None), (None, hi), (None, None)):
        assert_same_codes(port.clip(x, x_dt, lo_, b_dt, hi_, b_dt, out_dt), ref.clip(x, x_dt, lo_, b_dt, hi_, b_dt, out_dt), out_dt)
    if b_dt == "float32":                                    # a NaN bound leaves the values alone
        nan = np.array([np.nan], np.float32)
        assert_same_codes(port.clip(x, x_dt, nan, b_dt, hi, b_dt, out_dt), ref.clip(x, x_dt, nan, b_dt, hi, b_dt, out_dt), out_dt)


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (2, 3, 9, 8), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float16", "float16", (1, 4, 12, 12), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("int8", "int8", (2, 2, 7, 7), (3, 2), (1, 0, 1, 1), (1, 2), (1, 1)),
    ("bfloat16", "float32", (1, 2, 10, 11), (3, 3), (2, 2, 2, 2), (1, 1), (2, 2)),
    ("float32", "float32", (1, 1, 3, 3), (2, 2), (2, 2, 2, 2), (3, 3), (1, 1)),          # windows made of padding only
    ("float64", "float64", (3, 5, 7, 7), (7, 7), (0, 0, 0, 0), (1, 1), (1, 1)),
], ids=lambda p: f"{p[0]}-{p[2]}-k{p[3]}")
@pytest.mark.parametrize("include_pad", [0, 1])
def test_average_pool(port, ref, plan, include_pad):
    x_dt, out_dt, xs, kernel, pads, strides, dil = plan
    rng = np.random.default_rng(23)
    x = make(rng, xs, x_dt)
    args = (x, x_dt, out_dt, kernel, pads, strides, dil, include_pad)
    assert_same_codes(port.average_pool(*args), ref.average_pool(*args), out_dt)


@pytest.mark.parametrize("plan", [("float32", "float32", (4, 6, 7, 7)), ("float16", "float16", (2, 3, 5, 9)), ("int8", "float32", (1, 8, 4, 4)),
                                  ("bfloat16", "bfloat16", (3, 2, 1, 1)), ("float32", "int32", (2, 2, 3, 3))], ids=lambda p: f"{p[0]}-{p[1]}")
def test_global_average_pool(port, ref, plan):
    x_dt, out_dt, xs = plan
    x = make(np.random.default_rng(31), xs, x_dt)
    assert_same_codes(port.global_average_pool(x, x_dt, out_dt), ref.global_average_pool(x, x_dt, out_dt), out_dt)


@pytest.mark.parametrize("plan", [("float32", "float32", "float32", (3, 5, 6, 7)), ("float16", "float32", "float16", (2, 4, 5, 5)),
                                  ("bfloat16", "bfloat16", "float32", (1, 3, 8, 2)), ("float64", "float64", "float64", (2, 2, 3, 3)),
                                  ("float32", "float32", "float32", (4, 6)), ("int8", "float32", "float32", (2, 3, 4, 4))],
                         ids=lambda p: f"{p[0]}-{p[1]}-{p[2]}-{len(p[3])}d")
def test_batch_norm(port, ref, plan):
    x_dt, p_dt, out_dt, xs = plan
    rng = np.random.default_rng(37)
    x = make(rng, xs, x_dt)
    c = xs[1]
    scale, bias, mean = (from_f64(rng.normal(0, 1, c), p_dt) for _ in range(3))
    var = from_f64(rng.uniform(0.1, 2.0, c), p_dt)
    for eps in (1e-5, 1e-3):
        args = (x, x_dt, scale, bias, mean, var, p_dt, out_dt, eps)
        assert_same_codes(port.batch_norm(*args), ref.batch_norm(*args), out_dt)


# ---- Max / Min / Pow and the one-line unary operators ----------------------------------------------------------------
@pytest.mark.parametrize("plan", [("float32", "float32", "float32"), ("float16", "float16", "float16"), ("bfloat16", "float32", "float32"),
                                  ("int8", "int8", "int8"), ("int32", "int32", "int32"), ("int32", "float16", "float64"), ("uint8", "int8", "int16"),
                                  ("int64", "int64", "int64"), ("float32", "float32", "int8"), ("float8_e4m3", "float8_e4m3", "float8_e4m3")], ids="-".join)
@pytest.mark.parametrize("op", ["max", "min", "pow"])
def test_max_min_pow(port, ref, op, plan):
    a_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32((op + "-".join(plan)).encode()))
    a, b = make(rng, (9, 31), a_dt), make(rng, (9, 31), b_dt)
    if a_dt == "float32":
        a.reshape(-1)[:6] = [np.nan, 1.0, np.inf, -np.inf, 0.0, -0.0]
        b.reshape(-1)[:6] = [1.0, np.nan, 1.0, 2.0, -0.0, 0.0]
    if op == "pow" and b_dt in ("float32", "float16", "bfloat16"):
        b = from_f64(np.clip(np.asarray(rng.normal(0, 1.5, b.shape)), -4, 4), b_dt)
    assert_same_codes(port.binary(op, a, a_dt, b, b_dt, out_dt), ref.binary(op, a, a_dt, b, b_dt, out_dt), out_dt, f"{op} {plan}")


@pytest.mark.parametrize("op", ["exp", "log", "sqrt", "sigmoid", "tanh", "neg", "reciprocal", "ceil", "floor", "sin", "tan", "atan", "softplus",
                                "softsign", "hard_swish", "acos", "asin", "cosh", "sinh", "asinh", "acosh", "atanh", "round", "erf", "gelu"])
def test_unary_math_family(port, ref, op):
    """Same libm on both sides: the restatement and the reference agree bit for bit."""
    rng = np.random.default_rng(zlib.crc32(op.encode()))
    for x_dt, out_dt in (("float32", "float32"), ("float16", "float16"), ("bfloat16", "float32"), ("float64", "float64"), ("int8", "float32"),
                         ("float32", "int32"), ("float8_e4m3", "float16")):
        x = make(rng, (7, 53), x_dt, -3, 3) if x_dt in FLOAT_DTYPES else make(rng, (7, 53), x_dt)
        if x_dt == "float32":
            x.reshape(-1)[:8] = [0.0, -0.0, 1.0, -1.0, 0.5, np.inf, -np.inf, np.nan]
        assert_same_codes(port.unary_math(op, x, x_dt, out_dt), ref.unary_math(op, x, x_dt, out_dt), out_dt, f"{op} {x_dt}->{out_dt}")


# ---- MatMul and DynamicQuantizeLinear --------------------------------------------------------------------------------
MATMUL_PLANS = [  # a_dt, b_dt, out_dt, a shape, b shape
    ("float32", "float32", "float32", (7, 13), (13, 5)),
    ("float32", "float32", "float32", (3, 2, 7, 13), (13, 5)),
    ("float16", "float16", "float16", (4, 6, 9), (4, 9, 11)),
    ("bfloat16", "float32", "float32", (2, 1, 6, 8), (1, 3, 8, 4)),
    ("float64", "float64", "float64", (5, 17), (2, 17, 3)),
    ("int8", "int8", "int32", (3, 5, 12), (12, 7)),
    ("int32", "float32", "float64", (1, 4, 6), (5, 6, 2)),
    ("float8_e4m3", "float8_e4m3", "float16", (2, 8, 16), (2, 16, 8)),
    ("float32", "float32", "int8", (1, 9), (9, 1)),
]


@pytest.mark.parametrize("plan", MATMUL_PLANS, ids=lambda p: f"{p[0]}-{p[1]}-{p[2]}-{len(p[3])}x{len(p[4])}")
def test_matmul(port, ref, plan):
    a_dt, b_dt, out_dt, a_shape, b_shape = plan
    rng = np.random.default_rng(zlib.crc32(repr(plan).encode()))
    a, b = make(rng, a_shape, a_dt), make(rng, b_shape, b_dt)
    assert_same_codes(port.matmul(a, a_dt, b, b_dt, out_dt), ref.matmul(a, a_dt, b, b_dt, out_dt), out_dt)


@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64", "int8", "float8_e5m2"])
def test_dynamic_quantize_linear(port, ref, x_dt):
    rng = np.random.default_rng(zlib.crc32(x_dt.encode()))
    cases = [make(rng, (5, 77), x_dt), np.abs(to_f64(make(rng, (300,), x_dt), x_dt)), -np.abs(to_f64(make(rng, (300,), x_dt), x_dt)),
             np.zeros((4, 4)), np.full((3,), 2.5), np.zeros((0,))]
    cases = [cases[0]] + [from_f64(c, x_dt) for c in cases[1:]]
    if x_dt == "float32":
        odd = make(rng, (64,), x_dt)
        odd[:3] = [np.nan, 1e30, -3.0]
        cases.append(odd)
        inf = make(rng, (16,), x_dt)
        inf[2], inf[5] = -np.inf, np.inf
        cases.append(inf)
        halves = (np.arange(-40, 41) * 0.5 * (10.0 / 255.0)).astype(np.float32)        # quotients at and near .5 ties
        cases.append(np.concatenate([halves, np.float32([-5.0, 5.0])]))
    for x in cases:
        got, want = port.dynamic_quantize_linear(x, x_dt), ref.dynamic_quantize_linear(x, x_dt)
        for g, w, dt in zip(got, want, ("uint8", "float32", "uint8")):
            assert_same_codes(g, w, dt)
    # other output types go through the ordinary store
    x = make(rng, (33,), x_dt)
    got, want = port.dynamic_quantize_linear(x, x_dt, "int16", "float64", "int32"), ref.dynamic_quantize_linear(x, x_dt, "int16", "float64", "int32")
    for g, w, dt in zip(got, want, ("int16", "float64", "int32")):
        assert_same_codes(g, w, dt)


def test_dynamic_quantize_halves_equal_the_whole(port, ref):
    """Range + apply (the split used when the rows live on several GPUs) reproduce the reference's single call."""
    rng = np.random.default_rng(77)
    for x_dt in ("float32", "float16", "int8"):
        x = make(rng, (13, 21), x_dt)
        want = ref.dynamic_quantize_linear(x, x_dt)
        got = port.dynamic_quantize_apply(x, x_dt, port.dynamic_quantize_range(x, x_dt))
        for g, w, dt in zip(got, want, ("uint8", "float32", "uint8")):
            assert_same_codes(g, w, dt)
        # two row blocks, ranges combined
        r0, r1 = port.dynamic_quantize_range(x[:6], x_dt), port.dynamic_quantize_range(x[6:], x_dt)
        both = np.array([min(r0[0], r1[0]), max(r0[1], r1[1])])
        y0, y1 = port.dynamic_quantize_apply(x[:6], x_dt, both), port.dynamic_quantize_apply(x[6:], x_dt, both)
        assert_same_codes(np.concatenate([y0[0], y1[0]]), want[0], "uint8")
        assert_same_codes(y0[1], want[1], "float32")
        assert_same_codes(y1[2], want[2], "uint8")
