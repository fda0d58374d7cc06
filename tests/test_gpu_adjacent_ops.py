"""Cast, Clip, AveragePool, GlobalAveragePool and BatchNormalization on the GPU against the oracle: same
arithmetic in the same order, so every output code must be identical (any NaN equals any NaN)."""
import zlib

import numpy as np
import pytest

import gpu_ops as gpu
from datagen import ALL_DTYPES, FLOAT_DTYPES, assert_same_codes, from_f64, make

pytestmark = pytest.mark.gpu

OUT_SAMPLE = ("float8_e4m3", "float8_e5m2", "float16", "bfloat16", "float32", "float64", "int4", "int8", "uint8", "int16", "int32", "int64")
EDGE = np.array([0.0, -0.0, 0.5, 1.5, 2.5, -2.5, 127.4, 127.5, 128.5, -128.5, 255.5, 448.0, 465.0, 57344.0, 61440.0, 65504.0, 65520.0,
                 2.0 ** -6 * 0.999, 2.0 ** -14 * 0.999, 2.0 ** -24, 2.0 ** -25, 1e-40, 3e38, -3e38, 2147483648.0, -2147483649.0, 9.3e18,
                 -9.3e18, np.inf, -np.inf, np.nan])


@pytest.mark.parametrize("x_dt", ALL_DTYPES)
def test_cast_all_dtype_pairs(port, x_dt):
    rng = np.random.default_rng(zlib.crc32(f"gcast{x_dt}".encode()))
    x = make(rng, (41, 23), x_dt)
    if x_dt in FLOAT_DTYPES and x_dt not in ("float8_e4m3", "float8_e5m2"):
        with np.errstate(over="ignore", invalid="ignore"):
            x.reshape(-1)[:EDGE.size] = from_f64(EDGE, x_dt)
    for out_dt in OUT_SAMPLE:
        assert_same_codes(gpu.cast(x, x_dt, out_dt), port.cast(x, x_dt, out_dt), out_dt, f"cast {x_dt}->{out_dt}")


def test_cast_large_typed_pairs(port):
    rng = np.random.default_rng(5)
    x = rng.uniform(-300, 300, (257, 1031)).astype(np.float32)
    for out_dt in ("float16", "bfloat16", "int32", "int8", "int64", "float32"):
        assert_same_codes(gpu.cast(x, "float32", out_dt), port.cast(x, "float32", out_dt), out_dt)
    h = x.astype(np.float16)
    assert_same_codes(gpu.cast(h, "float16", "float32"), port.cast(h, "float16", "float32"), "float32")


@pytest.mark.parametrize("plan", [("float32", "float32", "float32"), ("float16", "float32", "float16"), ("int8", "int8", "int8"),
                                  ("int32", "float32", "int32"), ("bfloat16", "bfloat16", "float32"), ("float64", "float64", "float64"),
                                  ("float8_e4m3", "float32", "float8_e4m3"), ("uint8", "uint8", "int16")], ids="-".join)
def test_clip(port, plan):
    x_dt, b_dt, out_dt = plan
    rng = np.random.default_rng(zlib.crc32("gclip".encode() + "-".join(plan).encode()))
    x = make(rng, (6, 5, 70), x_dt)
    if x_dt in ("float32", "float64"):
        x.reshape(-1)[:4] = [np.nan, np.inf, -np.inf, -0.0]
    lo = from_f64(np.array([-3.0]), b_dt) if b_dt != "uint8" else np.array([2], np.uint8)
    hi = from_f64(np.array([5.0]), b_dt) if b_dt != "uint8" else np.array([9], np.uint8)
    for lo_, hi_ in ((lo, hi), (lo, None), (None, hi), (None, None)):
        assert_same_codes(gpu.clip(x, x_dt, lo_, b_dt, hi_, b_dt, out_dt), port.clip(x, x_dt, lo_, b_dt, hi_, b_dt, out_dt), out_dt)
    # bounds that vary per channel broadcast inside the kernel
    lo_c = np.ascontiguousarray(np.broadcast_to(lo, (5, 1))) if b_dt != "uint8" else np.full((5, 1), 2, np.uint8)
    assert_same_codes(gpu.clip(x, x_dt, lo_c, b_dt, hi, b_dt, out_dt), port.clip(x, x_dt, lo_c, b_dt, hi, b_dt, out_dt), out_dt)
    if b_dt == "float32":
        nan = np.array([np.nan], np.float32)
        assert_same_codes(gpu.clip(x, x_dt, nan, b_dt, hi, b_dt, out_dt), port.clip(x, x_dt, nan, b_dt, hi, b_dt, out_dt), out_dt)


@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16"])
def test_clip_same_type_with_scalar_bounds_of_any_type(port, x_dt):
    rng = np.random.default_rng(zlib.crc32(x_dt.encode()))
    for n in (1001, 4096, 7):
        x = make(rng, (n,), x_dt)
        for b_dt, lo, hi in (("float32", -0.75, 1.25), ("float16", -0.5, 0.5), ("int8", -1, 2), ("float64", -0.1, 0.3), ("float32", 0.0, -0.0)):
            lo_, hi_ = from_f64(np.array([lo]), b_dt), from_f64(np.array([hi]), b_dt)
            assert_same_codes(gpu.clip(x, x_dt, lo_, b_dt, hi_, b_dt, x_dt), port.clip(x, x_dt, lo_, b_dt, hi_, b_dt, x_dt), x_dt, f"{n} {b_dt}")


@pytest.mark.parametrize("plan", [
    ("float32", "float32", (2, 3, 9, 8), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float16", "float16", (1, 4, 12, 12), (2, 2), (0, 0, 0, 0), (2, 2), (1, 1)),
    ("int8", "int8", (2, 2, 7, 7), (3, 2), (1, 0, 1, 1), (1, 2), (1, 1)),
    ("bfloat16", "float32", (1, 2, 10, 11), (3, 3), (2, 2, 2, 2), (1, 1), (2, 2)),
    ("float32", "float32", (1, 1, 3, 3), (2, 2), (2, 2, 2, 2), (3, 3), (1, 1)),
    ("float32", "float32", (8, 64, 56, 56), (3, 3), (1, 1, 1, 1), (2, 2), (1, 1)),
    ("float32", "float32", (4, 256, 7, 7), (7, 7), (0, 0, 0, 0), (1, 1), (1, 1)),
], ids=lambda p: f"{p[0]}-{p[2]}-k{p[3]}")
@pytest.mark.parametrize("include_pad", [0, 1])
def test_average_pool(port, plan, include_pad):
    x_dt, out_dt, xs, kernel, pads, strides, dil = plan
    x = make(np.random.default_rng(23), xs, x_dt)
    args = (x, x_dt, out_dt, kernel, pads, strides, dil, include_pad)
    assert_same_codes(gpu.average_pool(*args), port.average_pool(*args), out_dt)


@pytest.mark.parametrize("plan", [("float32", "float32", (4, 6, 7, 7)), ("float16", "float16", (2, 3, 5, 9)), ("int8", "float32", (1, 8, 4, 4)),
                                  ("bfloat16", "bfloat16", (3, 2, 1, 1)), ("float32", "int32", (2, 2, 3, 3)), ("float32", "float32", (16, 2048, 7, 7)),
                                  ("float32", "float32", (2, 3, 112, 112)), ("float16", "float16", (2, 3, 20, 13)), ("bfloat16", "float32", (5, 7, 16, 8)),
                                  ("float32", "float16", (1, 1, 129, 1))], ids=lambda p: f"{p[0]}-{p[1]}-{p[2]}")
def test_global_average_pool(port, plan):
    x_dt, out_dt, xs = plan
    x = make(np.random.default_rng(31), xs, x_dt)
    assert_same_codes(gpu.global_average_pool(x, x_dt, out_dt), port.global_average_pool(x, x_dt, out_dt), out_dt)


@pytest.mark.parametrize("plan", [("float32", "float32", "float32", (3, 5, 6, 7)), ("float16", "float32", "float16", (2, 4, 5, 5)),
                                  ("bfloat16", "bfloat16", "float32", (1, 3, 8, 2)), ("float64", "float64", "float64", (2, 2, 3, 3)),
                                  ("float32", "float32", "float32", (4, 6)), ("int8", "float32", "float32", (2, 3, 4, 4)),
                                  ("float32", "float32", "float32", (8, 64, 56, 56)), ("float16", "float32", "float16", (2, 4, 8, 8)),
                                  ("bfloat16", "bfloat16", "bfloat16", (2, 3, 4, 16)), ("float32", "float64", "float32", (1, 2, 4))],
                         ids=lambda p: f"{p[0]}-{p[1]}-{p[2]}-{p[3]}")
def test_batch_norm(port, plan):
    x_dt, p_dt, out_dt, xs = plan
    rng = np.random.default_rng(37)
    x = make(rng, xs, x_dt)
    c = xs[1]
    scale, bias, mean = (from_f64(rng.normal(0, 1, c), p_dt) for _ in range(3))
    var = from_f64(rng.uniform(0.1, 2.0, c), p_dt)
    for eps in (1e-5, 1e-3):
        args = (x, x_dt, scale, bias, mean, var, p_dt, out_dt, eps)
        assert_same_codes(gpu.batch_norm(*args), port.batch_norm(*args), out_dt)


def test_adjacent_ops_reject_bad_arguments():
    from onnx_translator_b200 import capi
    with pytest.raises(capi.TensorOpsError):
        gpu.global_average_pool(np.zeros((2, 3, 4), np.float32), "float32", "float32")          # not 4-D
    with pytest.raises(capi.TensorOpsError):
        gpu.batch_norm(np.zeros((2, 5, 3), np.float32), "float32", *(np.ones(3, np.float32),) * 4, "float32", "float32")   # 3 < C
