"""GPU parity: every hot-path operator, called through the C ABI (via the package's operator
classes), against the CPU oracle on the same seeded inputs.

Bars (stated per test): bit-exact output codes for integer work, Q codes, MaxPool, Relu/Abs, DQ,
Add/Sub/Mul/Div, Cos (against the reference's TABLE cosine) and for Gemm/Conv on the exact path;
float32 relative tolerance 1e-6 for Softmax.  Any NaN equals any NaN.
"""
import zlib

import numpy as np
import pytest

import gpu_ops as gpu
from datagen import ALL_DTYPES, FLOAT_DTYPES, INT_DTYPES, assert_same_codes, from_f64, make, to_f64
from test_oracle_pin import BINARY_PLANS, CONV_PLANS, GEMM_PLANS, OUT_SAMPLE, _special_values

pytestmark = pytest.mark.gpu


def _seed(*parts):
    return zlib.crc32(repr(parts).encode())


# ---- unary -------------------------------------------------------------------------------------------
@pytest.mark.parametrize("x_dt", ALL_DTYPES)
@pytest.mark.parametrize("op", ["relu", "abs"])
def test_unary_all_dtype_pairs(port, op, x_dt):
    rng = np.random.default_rng(_seed(op, x_dt))
    x = make(rng, (37, 29), x_dt)
    if x_dt in FLOAT_DTYPES and x_dt not in ("float8_e4m3", "float8_e5m2"):
        with np.errstate(over="ignore", invalid="ignore"):
            x.reshape(-1)[:51] = from_f64(_special_values(x_dt), x_dt)
    for out_dt in OUT_SAMPLE:
        assert_same_codes(gpu.unary(op, x, x_dt, out_dt), port.unary(op, x, x_dt, out_dt), out_dt, f"{op} {x_dt}->{out_dt}")


@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64", "int8", "int32", "float8_e5m2"])
def test_cos_matches_reference_table_bit_for_bit(port, x_dt):
    rng = np.random.default_rng(7)
    if x_dt == "float8_e5m2":
        x = rng.integers(0, 0x7C, size=4096, dtype=np.uint8) | (rng.integers(0, 2, size=4096, dtype=np.uint8) << 7)
    else:
        x = np.concatenate([rng.uniform(-10, 10, 200000), rng.uniform(-1e4, 1e4, 50000),
                            [0.0, -0.0, 2 * np.pi, 4 * np.pi, 6.283185307179586, 6.2831854820251465,
                             12.566370614359172, 1e30, -1e30, 1e-30]])
        if x_dt == "float16":
            x = np.clip(x, -60000, 60000)
        x = from_f64(x if x_dt not in INT_DTYPES else np.clip(x, -120, 120), x_dt)
    for out_dt in ("float32", "float16", "bfloat16", "float64", "int8"):
        assert_same_codes(gpu.unary("cos", x, x_dt, out_dt), port.unary("cos", x, x_dt, out_dt), out_dt, f"cos {x_dt}->{out_dt}")


def test_unary_odd_sizes_and_empty(port):
    rng = np.random.default_rng(3)
    for n in (1, 3, 4, 5, 15, 16, 17, 255, 257, 1023, 4099):
        x = make(rng, (n,), "float32")
        assert_same_codes(gpu.unary("relu", x, "float32", "float32"), port.unary("relu", x, "float32", "float32"), "float32")
        xi = make(rng, (n,), "int8")
        assert_same_codes(gpu.unary("abs", xi, "int8", "int8"), port.unary("abs", xi, "int8", "int8"), "int8")
    assert gpu.unary("relu", np.zeros((0, 4), np.float32), "float32", "float32").shape == (0, 4)


# ---- binary ------------------------------------------------------------------------------------------
@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
@pytest.mark.parametrize("plan", BINARY_PLANS, ids=lambda p: "-".join(p))
def test_binary_same_shape(port, op, plan):
    a_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(_seed(op, plan))
    a = make(rng, (64, 67), a_dt)
    b = make(rng, (64, 67), b_dt)
    if b_dt in INT_DTYPES:
        b.reshape(-1)[::97] = 0
    assert_same_codes(gpu.binary(op, a, a_dt, b, b_dt, out_dt), port.binary(op, a, a_dt, b, b_dt, out_dt), out_dt, f"{op} {plan}")


BROADCAST_SHAPES = [
    ((10, 10, 10), (10, 1)), ((4, 1, 16), (16,)), ((8, 32, 64), (1, 32, 1)), ((8, 32, 64), (64,)),
    ((64,), (8, 32, 64)), ((5, 7, 3), (7, 1)), ((33,), (1,)), ((4, 1, 5), (1, 3, 1)), ((2, 16, 14, 14), (16, 1, 1)),
    ((2, 3, 4, 5, 6), (3, 1, 5, 1)), ((1, 1), (6, 7)), ((3, 1, 2, 1, 2, 1, 3), (1, 2, 1, 2, 1, 2, 1)),
]


@pytest.mark.parametrize("dts", [("float32", "float32", "float32"), ("int8", "int8", "int8"), ("bfloat16", "bfloat16", "bfloat16"),
                                 ("int8", "float32", "float32"), ("int32", "float16", "float64"), ("float16", "int16", "uint8")],
                         ids=lambda p: "-".join(p))
@pytest.mark.parametrize("shapes", BROADCAST_SHAPES, ids=lambda s: f"{s[0]}x{s[1]}")
def test_binary_broadcast(port, shapes, dts):
    a_dt, b_dt, out_dt = dts
    rng = np.random.default_rng(_seed(shapes, dts))
    a = make(rng, shapes[0], a_dt)
    b = make(rng, shapes[1], b_dt)
    for op in ("add", "sub", "mul", "div"):
        assert_same_codes(gpu.binary(op, a, a_dt, b, b_dt, out_dt), port.binary(op, a, a_dt, b, b_dt, out_dt), out_dt,
                          f"{op} {shapes} {dts}")


@pytest.mark.parametrize("op", ["add", "sub", "mul", "div"])
def test_binary_saturation_and_wrap(port, op):
    a = np.array([127, -128, 100, -100, 127, -128, 0, 1], dtype=np.int8)
    b = np.array([127, -128, 100, 100, -1, -1, 0, 0], dtype=np.int8)
    assert_same_codes(gpu.binary(op, a, "int8", b, "int8", "int8"), port.binary(op, a, "int8", b, "int8", "int8"), "int8")
    a32 = np.array([2 ** 31 - 1, -2 ** 31, 2 ** 31 - 1, 65536, -2 ** 31, 7, -7, 0], dtype=np.int32)
    b32 = np.array([2 ** 31 - 1, -2 ** 31, -2 ** 31, 65536, -1, 0, 0, 0], dtype=np.int32)
    for out in ("int32", "int64", "int16", "uint8"):
        assert_same_codes(gpu.binary(op, a32, "int32", b32, "int32", out), port.binary(op, a32, "int32", b32, "int32", out), out)
    a64 = np.array([2 ** 62, -2 ** 62, 2 ** 63 - 1, 3, 2 ** 40], dtype=np.int64)
    b64 = np.array([2 ** 62, -2 ** 62, 2, 0, 2 ** 40], dtype=np.int64)
    assert_same_codes(gpu.binary(op, a64, "int64", b64, "int64", "int64"), port.binary(op, a64, "int64", b64, "int64", "int64"), "int64")
    af = np.array([np.nan, np.inf, -np.inf, 1e30, -1e30, 2.5, 3.5, -2.5, 0.5, 1e10], dtype=np.float32)
    bf = np.ones(10, dtype=np.float32)
    for out in ("int8", "uint8", "int32", "int64", "int4"):
        assert_same_codes(gpu.binary(op, af, "float32", bf, "float32", out), port.binary(op, af, "float32", bf, "float32", out), out)


def test_narrow_integer_division_is_exact(port):
    """Division of 8- and 16-bit integers runs on a float reciprocal: every int8 and uint8 pair, and
    for int16 the pairs that stress it (exact multiples and their neighbours, extremes, random)."""
    a8, b8 = np.meshgrid(np.arange(-128, 128, dtype=np.int8), np.arange(-128, 128, dtype=np.int8), indexing="ij")
    for out in ("int8", "int16", "int32"):
        assert_same_codes(gpu.binary("div", a8.copy(), "int8", b8.copy(), "int8", out), port.binary("div", a8.copy(), "int8", b8.copy(), "int8", out), out)
    au, bu = np.meshgrid(np.arange(256, dtype=np.uint8), np.arange(256, dtype=np.uint8), indexing="ij")
    assert_same_codes(gpu.binary("div", au.copy(), "uint8", bu.copy(), "uint8", "uint8"), port.binary("div", au.copy(), "uint8", bu.copy(), "uint8", "uint8"), "uint8")
    assert_same_codes(gpu.binary("div", a8.copy(), "int8", bu.copy(), "uint8", "int16"), port.binary("div", a8.copy(), "int8", bu.copy(), "uint8", "int16"), "int16")
    rng = np.random.default_rng(41)
    b = rng.integers(-32768, 32768, size=1 << 20, dtype=np.int64)
    q = rng.integers(-40, 41, size=b.size, dtype=np.int64)
    near = np.clip(q * b + rng.integers(-1, 2, size=b.size), -32768, 32767)        # multiples of b and their neighbours
    rand = rng.integers(-32768, 32768, size=b.size, dtype=np.int64)
    edge = rng.choice(np.array([-32768, -32767, -1, 0, 1, 32767]), size=b.size)
    for a in (near, rand, edge):
        a16, b16 = a.astype(np.int16), b.astype(np.int16)
        for out in ("int16", "int32"):
            assert_same_codes(gpu.binary("div", a16, "int16", b16, "int16", out), port.binary("div", a16, "int16", b16, "int16", out), out)
    a16, b16 = edge.astype(np.int16), rng.choice(np.array([-32768, -1, 1, 2, 32767, 0]), size=b.size).astype(np.int16)
    assert_same_codes(gpu.binary("div", a16, "int16", b16, "int16", "int16"), port.binary("div", a16, "int16", b16, "int16", "int16"), "int16")


def test_binary_output_dtype_inference():
    """No explicit dtype: numpy promotion over the storage types (bfloat16 is stored as uint16)."""
    from onnx_translator_b200 import nn
    from onnx_translator_b200.nn import Operators as ops
    cases = [("float32", "float32", "float32"), ("float16", "float16", "float16"), ("bfloat16", "bfloat16", "bfloat16"),
             ("int32", "int32", "int32"), ("int8", "int8", "int8"), ("int8", "float32", "float32"),
             ("int32", "float16", "float64"), ("int8", "int32", "int32"), ("uint8", "int8", "int16"),
             ("int64", "float32", "float64"), ("bfloat16", "float32", "float32"), ("bfloat16", "float16", "float32")]
    for a_dt, b_dt, want in cases:
        a = nn.Tensor(4, dtype=a_dt)
        b = nn.Tensor(4, dtype=b_dt)
        out = ops.ADD([], [], dtype=None).forward(a, b)["tensor"]
        assert out.dtype == want, (a_dt, b_dt, out.dtype)


def test_binary_incompatible_shapes_raise():
    from onnx_translator_b200 import nn
    from onnx_translator_b200.nn import Operators as ops
    with pytest.raises(ValueError):
        ops.ADD([], [], dtype="float32").forward(nn.Tensor(3, 4), nn.Tensor(5,))


def test_full_size_add_matches_ieee_float32():
    """BASELINE config 2 at full size: A[64,512,1024] (+) B[1,512,1] in float32.  numpy's float32
    arithmetic is IEEE and serves as the size-independent check."""
    rng = np.random.default_rng(0)
    a = rng.uniform(-100, 100, (64, 512, 1024)).astype(np.float32)
    b = (rng.uniform(0.5, 100, (1, 512, 1)) * rng.choice([-1, 1], (1, 512, 1))).astype(np.float32)
    for op, fn in (("add", np.add), ("sub", np.subtract), ("mul", np.multiply), ("div", np.divide)):
        got = gpu.binary(op, a, "float32", b, "float32", "float32")
        assert np.array_equal(got, fn(a, b)), op


# ---- quantize / dequantize ------------------------------------------------------------------------------
@pytest.mark.parametrize("out_dt", ["int8", "uint8", "int4", "int16", "int32", "float8_e4m3", "float8_e5m2", "float16", "float32"])
@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64"])
def test_quantize(port, x_dt, out_dt):
    rng = np.random.default_rng(11)
    x = make(rng, (2, 16, 12, 12), x_dt)
    zp_dt = out_dt if out_dt in INT_DTYPES else "int8"
    s = np.array([0.02], dtype=np.float32)
    z = np.array([3], dtype=np.int64).astype(np.int8 if zp_dt != "uint8" else np.uint8)
    assert_same_codes(gpu.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt), port.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt), out_dt, "per-tensor")
    s = rng.uniform(0.01, 0.05, 16).astype(np.float32)
    s[5] = 0.0
    z = rng.integers(0, 9, 16).astype(z.dtype)
    assert_same_codes(gpu.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt, axis=1),
                      port.quantize(x, x_dt, s, "float32", z, zp_dt, out_dt, axis=1), out_dt, "per-axis")
    # full-size scale / zero point, as the reference's own caller passes them
    sf = np.broadcast_to(s.reshape(1, 16, 1, 1), x.shape).copy()
    zf = np.broadcast_to(z.reshape(1, 16, 1, 1), x.shape).copy()
    assert_same_codes(gpu.quantize(x, x_dt, sf, "float32", zf, zp_dt, out_dt), port.quantize(x, x_dt, sf, "float32", zf, zp_dt, out_dt), out_dt, "full-size")


def test_quantize_edge_values(port):
    x = np.array([0.49, 0.5, 0.51, 1.5, 2.5, -0.5, -1.5, 17.3, 1e9, -1e9, np.inf, -np.inf, np.nan,
                  2.55, 2.56, -2.57, 448 / 16, 449, 1e-9, 60000.0, 70000.0, 0.03, 0.01, -0.05], dtype=np.float32)
    for out_dt, zp_dt, zp in (("int8", "int8", 0), ("uint8", "uint8", 128), ("float8_e4m3", "int8", 0), ("float8_e4m3", "float8_e4m3", 0),
                              ("float8_e5m2", "int8", 0), ("float8_e5m2", "float8_e5m2", 0), ("int32", "int32", 5)):
        for s in (1.0, 0.02, 1 / 16, 3.0, 0.0):
            sv = np.array([s], dtype=np.float32)
            zv = np.array([zp]).astype(np.uint8 if zp_dt in ("uint8", "float8_e4m3", "float8_e5m2") else np.int32)
            assert_same_codes(gpu.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt),
                              port.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt), out_dt, f"{out_dt} s={s}")


def test_quantize_with_scales_at_the_ends_of_the_float_range(port):
    """Scales whose reciprocal is subnormal or infinite in float32: the approximate reciprocal is useless
    there and every element has to reach the exact division."""
    x = np.tile(np.array([3e38, -3e38, 1.2e38, 0.0, 1e-40, -2e-45, 1.0, 2.9e-39, np.inf], dtype=np.float32), 40)
    for out_dt, zp_dt, zp in (("int8", "int8", 1), ("uint8", "uint8", 128), ("float8_e4m3", "int8", 0), ("int32", "int32", 5)):
        for s in (1e38, 1.7e38, 8.6e37, 8.4e37, 1e-39, 1.4e-45, 2e-38):
            sv = np.array([s], dtype=np.float32)
            zv = np.array([zp]).astype(np.uint8 if zp_dt == "uint8" else np.int32)
            assert_same_codes(gpu.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt),
                              port.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt), out_dt, f"{out_dt} s={s}")
        per_axis = np.array([1e38, 1e-39, 0.5, 1.7e38, 0.0, 8.6e37, 3.0, 1e-3], dtype=np.float32)
        xa = np.tile(x[:9], (8, 5)).astype(np.float32)
        za = np.full(8, zp).astype(np.uint8 if zp_dt == "uint8" else np.int32)
        assert_same_codes(gpu.quantize(xa, "float32", per_axis, "float32", za, zp_dt, out_dt, axis=0),
                          port.quantize(xa, "float32", per_axis, "float32", za, zp_dt, out_dt, axis=0), out_dt, f"{out_dt} per axis")


@pytest.mark.parametrize("cfg", [("int8", 0.02, 0), ("uint8", 0.02, 128), ("float8_e4m3", 1 / 16, 0), ("float8_e5m2", 1 / 16, 0)],
                         ids=lambda c: c[0])
def test_quantize_near_ties_against_double_division(port, cfg):
    """x chosen so that x / s sits within a few float ulps of k + 0.5: the fast float path must
    hand exactly these to the double division."""
    out_dt, s, zp = cfg
    rng = np.random.default_rng(5)
    k = rng.integers(-120, 120, 200000)
    s32 = np.float32(s)
    mid = ((k + 0.5) * np.float64(s32)).astype(np.float32)
    x = np.concatenate([mid, np.nextafter(mid, np.float32(np.inf)), np.nextafter(mid, np.float32(-np.inf))])
    zp_dt = out_dt if out_dt in ("int8", "uint8") else "int8"
    zv = np.array([zp]).astype(np.uint8 if zp_dt == "uint8" else np.int8)
    sv = np.array([s32])
    assert_same_codes(gpu.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt),
                      port.quantize(x, "float32", sv, "float32", zv, zp_dt, out_dt), out_dt)


@pytest.mark.parametrize("x_dt", ["int8", "uint8", "int32", "float8_e4m3", "float8_e5m2", "int4", "int16"])
@pytest.mark.parametrize("out_dt", ["float32", "float16", "bfloat16", "float64"])
def test_dequantize(port, x_dt, out_dt):
    rng = np.random.default_rng(13)
    x = make(rng, (3, 8, 10, 10), x_dt)
    z = make(rng, (1,), x_dt) if x_dt not in ("float8_e4m3", "float8_e5m2") else np.array([0], dtype=np.uint8)
    s = np.array([0.0173], dtype=np.float32)
    assert_same_codes(gpu.dequantize(x, x_dt, s, "float32", z, x_dt, out_dt), port.dequantize(x, x_dt, s, "float32", z, x_dt, out_dt), out_dt)
    s = rng.uniform(0.005, 0.02, (1, 8, 1, 1)).astype(np.float32)
    zb = np.broadcast_to(z, (1, 8, 1, 1)).copy()
    assert_same_codes(gpu.dequantize(x, x_dt, s, "float32", zb, x_dt, out_dt), port.dequantize(x, x_dt, s, "float32", zb, x_dt, out_dt), out_dt)
    if x_dt in ("float8_e4m3", "float8_e5m2"):        # non-zero fp8 zero point: the difference needs double for e5m2
        zc = np.array([0x3A], dtype=np.uint8)
        assert_same_codes(gpu.dequantize(x, x_dt, s, "float32", zc, x_dt, out_dt), port.dequantize(x, x_dt, s, "float32", zc, x_dt, out_dt), out_dt)


def test_qdq_roundtrip_config3_rows(port):
    """BASELINE config 3 on a 512 x 8192 slab (same distribution and scales as the 8192^2 case)."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((512, 8192)).astype(np.float32)
    s_axis = rng.uniform(0.01, 0.05, 8192).astype(np.float32)
    z_axis = rng.integers(-8, 9, 8192).astype(np.int8)
    plans = [("int8", np.array([0.02], np.float32), np.array([0], np.int8), "int8", None),
             ("uint8", np.array([0.02], np.float32), np.array([128], np.uint8), "uint8", None),
             ("int8", s_axis, z_axis, "int8", 1),
             ("float8_e4m3", np.array([1 / 16], np.float32), np.array([0], np.int8), "int8", None),
             ("float8_e5m2", np.array([1 / 16], np.float32), np.array([0], np.int8), "int8", None)]
    for out_dt, s, z, z_dt, axis in plans:
        q_gpu = gpu.quantize(x, "float32", s, "float32", z, z_dt, out_dt, axis=axis)
        q_cpu = port.quantize(x, "float32", s, "float32", z, z_dt, out_dt, axis=axis)
        assert_same_codes(q_gpu, q_cpu, out_dt, f"Q {out_dt}")
        sb = s if axis is None else s.reshape(1, -1)
        zb = z if axis is None else z.reshape(1, -1)
        assert_same_codes(gpu.dequantize(q_gpu, out_dt, sb, "float32", zb, z_dt, "float32"),
                          port.dequantize(q_cpu, out_dt, sb, "float32", zb, z_dt, "float32"), "float32", f"DQ {out_dt}")


def test_full_size_quantize_matches_double_formula():
    """8192 x 8192 float32 -> int8 at full size against the formula evaluated in numpy float64."""
    rng = np.random.default_rng(0)
    x = rng.standard_normal((8192, 8192)).astype(np.float32)
    s = np.float32(0.02)
    got = gpu.quantize(x, "float32", np.array([s]), "float32", np.array([0], np.int8), "int8", "int8")
    want = np.clip(np.rint(x.astype(np.float64) / np.float64(s)), -128, 127).astype(np.int8)
    assert np.array_equal(got, want)
    back = gpu.dequantize(got, "int8", np.array([s]), "float32", np.array([0], np.int8), "int8", "float32")
    assert np.array_equal(back, (want.astype(np.float64) * np.float64(s)).astype(np.float32))


# ---- conv / pool / gemm / softmax / flatten -----------------------------------------------------------------
@pytest.mark.parametrize("plan", CONV_PLANS, ids=lambda p: f"{p[0]}-{p[3]}-g{p[9]}")
def test_conv2d_exact_path(port, plan):
    x_dt, w_dt, b_dt, out_dt, xs, ws, pads, strides, dil, group = plan
    rng = np.random.default_rng(17)
    x = make(rng, xs, x_dt, -2, 2) if x_dt not in INT_DTYPES else make(rng, xs, x_dt)
    w = make(rng, ws, w_dt, -1, 1) if w_dt not in INT_DTYPES else make(rng, ws, w_dt)
    b = None if b_dt is None else make(rng, (ws[0],), b_dt)
    args = (x, x_dt, w, w_dt, b, b_dt or "float32", out_dt, pads, strides, dil, group)
    assert_same_codes(gpu.conv2d(*args), port.conv2d(*args), out_dt)


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (1, 1, 4, 4), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("bfloat16", "bfloat16", (2, 3, 16, 16), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("float32", "float32", (2, 4, 15, 14), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float16", "float32", (1, 2, 12, 12), (3, 2), (2, 0, 1, 1), (1, 2), (2, 2)),
    ("int8", "int8", (1, 2, 9, 9), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float8_e4m3", "float8_e4m3", (1, 2, 9, 9), (2, 2), (0, 0, 0, 0), (1, 1), (1, 1)),
    ("float32", "float32", (1, 1, 3, 3), (2, 2), (2, 2, 2, 2), (3, 3), (1, 1)),
    ("float32", "float32", (4, 64, 112, 112), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),      # the ResNet stem pool
    ("float32", "float32", (4, 256, 7, 7), (7, 7), (0, 0, 0, 0), (1, 1), (1, 1)),          # the final 7x7 pool
    ("float16", "float16", (3, 5, 24, 40), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("bfloat16", "bfloat16", (2, 7, 34, 132), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("int8", "int8", (2, 3, 18, 20), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float32", "float32", (3, 9, 6, 8), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("uint8", "uint8", (1, 130, 8, 136), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("float8_e5m2", "float8_e5m2", (2, 2, 10, 12), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
], ids=lambda p: f"{p[0]}-{p[2]}-k{p[3]}")
def test_max_pool(port, plan):
    x_dt, out_dt, xs, kernel, pads, strides, dil = plan
    rng = np.random.default_rng(19)
    x = make(rng, xs, x_dt)
    if x_dt == "float32":
        x.reshape(-1)[::7] = np.nan
        x.reshape(-1)[3::11] = -np.inf
        x.reshape(-1)[1::5] = 0.0                  # ties between +0 and -0 go to the first tap scanned
        x.reshape(-1)[2::5] = -0.0
        x.reshape(-1)[4::10] = -1.0
    args = (x, x_dt, out_dt, kernel, pads, strides, dil)
    assert_same_codes(gpu.max_pool(*args), port.max_pool(*args), out_dt)


@pytest.mark.parametrize("plan", GEMM_PLANS, ids=lambda p: f"{p[0]}-{p[3]}-{p[9]}{p[10]}")
def test_gemm_exact_path(port, plan):
    a_dt, b_dt, c_dt, out_dt, ash, bsh, csh, alpha, beta, ta, tb = plan
    rng = np.random.default_rng(23)
    a = make(rng, ash, a_dt, -2, 2) if a_dt not in INT_DTYPES else make(rng, ash, a_dt)
    b = make(rng, bsh, b_dt, -2, 2) if b_dt not in INT_DTYPES else make(rng, bsh, b_dt)
    c = None if c_dt is None else make(rng, csh, c_dt)
    args = (a, a_dt, b, b_dt, c, c_dt or "float32", out_dt, alpha, beta, ta, tb)
    assert_same_codes(gpu.gemm(*args), port.gemm(*args), out_dt)


def test_gemm_exact_path_float32_ragged_tiles(port):
    rng = np.random.default_rng(29)
    for (m, n, k, ta, tb) in [(130, 70, 257, 0, 1), (65, 129, 33, 1, 0), (1, 10, 4096, 0, 1), (200, 3, 17, 1, 1)]:
        a = rng.normal(0, 0.5, (k, m) if ta else (m, k)).astype(np.float32)
        b = rng.normal(0, 0.5, (n, k) if tb else (k, n)).astype(np.float32)
        c = rng.normal(0, 1, (n,)).astype(np.float32)
        args = (a, "float32", b, "float32", c, "float32", "float32", 1.0, 1.0, ta, tb)
        assert_same_codes(gpu.gemm(*args), port.gemm(*args), "float32", f"{m}x{n}x{k}")


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (2, 5), -1), ("float16", "float16", (4, 64), 1), ("float8_e4m3", "float8_e4m3", (2, 10), 1),
    ("float32", "float32", (3, 7, 5), 1), ("float32", "float32", (3, 7, 5), 0), ("bfloat16", "float32", (6, 1000), -1),
    ("float64", "float64", (5, 33), 1), ("float32", "float16", (2, 3, 4, 5), 2), ("float32", "float32", (64, 1000), 1),
    ("float32", "float32", (3, 5000), 1), ("float32", "float32", (2, 40000), 1), ("bfloat16", "bfloat16", (33, 777), 1),
    ("float32", "float32", (7, 999), 1), ("float32", "float32", (5, 1023), 1), ("float32", "float32", (3000, 16), 1),
    ("float16", "float16", (130, 1024), 1), ("bfloat16", "bfloat16", (64, 1000), 1), ("float16", "float16", (9, 18), 1),
    ("float32", "float32", (2500, 1024), 1), ("float32", "float32", (1, 20), 0),
], ids=lambda p: f"{p[0]}-{p[2]}-ax{p[3]}")
def test_softmax(port, plan):
    """Tolerance: |gpu - oracle| <= 1e-6 * |oracle| + one unit in the last place of the output type
    (the parallel sum adds in a different order than the sequential double sum; float32 / float16 /
    bfloat16 rows are evaluated in compensated float32).  Below the normal range one unit in the last
    place is the denormal step of the type (for float16 the reference's flush threshold 2^-24)."""
    x_dt, out_dt, shape, axis = plan
    rng = np.random.default_rng(29)
    if x_dt == "float8_e4m3":
        x = rng.integers(0, 0x7F, size=shape, dtype=np.uint8) | (rng.integers(0, 2, size=shape, dtype=np.uint8) << 7)
    else:
        x = make(rng, shape, x_dt)
    got = to_f64(gpu.softmax(x, x_dt, out_dt, axis), out_dt)
    want = to_f64(port.softmax(x, x_dt, out_dt, axis), out_dt)
    ulp = {"float32": 2.0 ** -23, "float64": 2.0 ** -52, "float16": 2.0 ** -10, "bfloat16": 2.0 ** -7, "float8_e4m3": 2.0 ** -3}[out_dt]
    step = {"float32": 2.0 ** -149, "float16": 2.0 ** -24, "bfloat16": 2.0 ** -133}.get(out_dt, 0.0) if x_dt == out_dt else 0.0
    assert np.all(np.abs(got - want) <= 1e-6 * np.abs(want) + ulp * np.abs(want) + step + 1e-45), np.max(np.abs(got - want))
    assert np.allclose(got.sum(axis=axis), 1.0, atol=1e-2 if out_dt != "float32" else 1e-5)


def test_flatten_copy_and_view(port):
    rng = np.random.default_rng(31)
    for dt in ("float32", "int8", "bfloat16", "float64"):
        x = make(rng, (2, 3, 4, 5), dt)
        assert_same_codes(gpu.flatten(x, dt, (2, 60), copy=True), port.flatten(x, dt, (2, 60)), dt)
        assert_same_codes(gpu.flatten(x, dt, (2, 60), copy=False), port.flatten(x, dt, (2, 60)), dt)


# ---- codecs and error reporting -------------------------------------------------------------------------------
@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float8_e4m3", "float8_e5m2"])
def test_encoder_exhaustive_on_device(dt):
    """All 2^32 float32 inputs: the hardware-convert encoder equals the bit-level restatement of
    the reference encoder (which test_codec_tables pins against the oracle)."""
    from onnx_translator_b200 import capi
    lib = capi.load()
    assert lib.tops_selftest_encoder(capi.DTYPE_MAP[dt]) == 0
    capi.check(lib)


@pytest.mark.parametrize("dt", ["float16", "bfloat16", "float8_e4m3", "float8_e5m2"])
def test_codec_tables(port, dt):
    """Decode every code; encode a dense float32 sweep (2^20 exponent/mantissa prefixes x 6 tails)."""
    nbits = 16 if dt in ("float16", "bfloat16") else 8
    codes = np.arange(2 ** nbits, dtype=np.uint32).astype(np.uint16 if nbits == 16 else np.uint8)
    if dt == "float16":
        codes = codes.view(np.float16)
    zero = np.zeros(codes.shape, dtype=np.float32)
    assert_same_codes(gpu.binary("add", codes, dt, zero, "float32", "float32"), port.binary("add", codes, dt, zero, "float32", "float32"), "float32", "decode")
    hi = np.arange(2 ** 20, dtype=np.uint32) << 12
    for low in (0x000, 0x001, 0x7FF, 0x800, 0x801, 0xFFF):
        x = (hi | np.uint32(low)).view(np.float32)
        assert_same_codes(gpu.unary("abs", x, "float32", dt), port.unary("abs", x, "float32", dt), dt, f"encode low={low:#x}")


def test_rejected_call_zero_fills_and_reports():
    """Size mismatch: the reference returns silently leaving calloc zeros; here the output is
    zero-filled and the error is retrievable."""
    import ctypes
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    a = DeviceArray.from_numpy(np.ones(8, np.float32), "float32")
    out = DeviceArray.from_numpy(np.full(5, 7.0, np.float32), "float32")
    lib.relu_forward(a.handle, out.handle)
    assert lib.tops_last_error() == 1
    lib.tops_clear_error()
    assert np.array_equal(out.numpy(), np.zeros(5, np.float32))
    lib.relu_forward(None, out.handle)
    assert lib.tops_last_error() == 1
    lib.tops_clear_error()


def test_create_tensor_is_zero_filled_and_views_share_memory():
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    z = DeviceArray.empty((3, 5), "int32", zero=True)
    assert np.array_equal(z.numpy(), np.zeros((3, 5), np.int32))
    x = DeviceArray.from_numpy(np.arange(24, dtype=np.float32).reshape(4, 6), "float32")
    v = x.reshape(2, 12)
    rows = x.rows(1, 2)
    del x                                             # views keep the allocation alive
    assert np.array_equal(v.numpy(), np.arange(24, dtype=np.float32).reshape(2, 12))
    assert np.array_equal(rows.numpy(), np.arange(6, 18, dtype=np.float32).reshape(2, 6))
    capi.check()


def test_fast_cosine_division_is_exact_for_every_float32():
    """All finite float32 inputs: multiply-by-reciprocal plus one fused correction gives the same
    double as the reference's multiply-then-divide."""
    from onnx_translator_b200 import capi
    lib = capi.load()
    assert lib.tops_selftest_cos() == 0
    capi.check(lib)


def test_cos_subnormal_huge_and_unaligned_inputs(port):
    x = np.array([1e-40, -1e-45, 1.1754944e-38, 0.0, 3.4e38, -3.4e38, 12.566371, 12.56637, 6.2831855, 6.283185,
                  100.0, -1000.5, 65504.0], dtype=np.float32)
    assert_same_codes(gpu.unary("cos", x, "float32", "float32"), port.unary("cos", x, "float32", "float32"), "float32")
    rng = np.random.default_rng(41)
    for n in (1, 3, 5, 7, 1023, 4097):
        for dt in ("float32", "float16", "bfloat16"):
            v = from_f64(rng.uniform(-20, 20, n), dt)
            assert_same_codes(gpu.unary("cos", v, dt, dt), port.unary("cos", v, dt, dt), dt, f"{dt} n={n}")
