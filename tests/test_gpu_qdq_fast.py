"""QuantizeLinear / DequantizeLinear through the dedicated loops for one scale per tensor and one per element of the
last dimension (csrc/qdq_fast.cu) against the oracle (tensor_ops.c:999-1034), bit for bit: rounding ties, values beyond
the saturation limits, NaN, infinities, a zero scale, tails that are not a multiple of 16, every 8-bit code type."""
import numpy as np
import pytest

import gpu_ops as gpu
from datagen import from_f64

pytestmark = pytest.mark.gpu

CODES = [("int8", "int8"), ("uint8", "uint8"), ("float8_e4m3", "int8"), ("float8_e5m2", "int8")]


def _values(rng, shape, scale):
    x = rng.normal(0, 1, shape).astype(np.float32)
    flat = x.reshape(-1)
    s = np.broadcast_to(scale, shape).reshape(-1)
    flat[::5] = ((np.rint(flat[::5] / s[::5]) + 0.5) * s[::5]).astype(np.float32)          # at and next to rounding ties
    flat[1::7] *= 400                                                                       # beyond the 8-bit range
    flat[2::29] = np.float32(3e38)
    flat[3::31] = np.float32(-np.inf)
    flat[4::37] = np.float32(np.nan)
    flat[6::41] = np.float32(np.inf)
    flat[8::43] = np.float32(2e6) * s[8::43]                                                # quotients past the e5m2 overflow threshold
    return x


def _same(got, want):
    return got.shape == want.shape and np.array_equal(got.view(np.uint8), want.view(np.uint8))


@pytest.mark.parametrize("codes", CODES, ids=lambda c: c[0])
@pytest.mark.parametrize("shape", [(64, 256), (7, 33), (3, 5, 48), (1, 16)], ids=str)
def test_per_tensor_forms(port, codes, shape):
    code_dt, zero_dt = codes
    rng = np.random.default_rng(shape[-1])
    for scale_value, zero_value in ((0.02, 0), (0.37, 5 if code_dt != "uint8" else 128), (0.0, 3)):
        scale = np.array([scale_value], np.float32)
        zero = np.array([zero_value], np.int8 if zero_dt == "int8" else np.uint8)
        x = _values(rng, shape, np.float32(scale_value if scale_value else 1.0))
        want = port.quantize(x, "float32", scale, "float32", zero, zero_dt, code_dt)
        got = gpu.quantize(x, "float32", scale, "float32", zero, zero_dt, code_dt)
        assert _same(got, want), (codes, shape, scale_value)
        all_codes = rng.integers(0, 256, shape).astype(np.uint8).view(want.dtype)
        back_want = port.dequantize(all_codes, code_dt, scale, "float32", zero, zero_dt, "float32")
        back = gpu.dequantize(all_codes, code_dt, scale, "float32", zero, zero_dt, "float32")
        nan = np.isnan(back_want)
        assert np.array_equal(np.isnan(back), nan) and np.array_equal(back[~nan].view(np.uint32), back_want[~nan].view(np.uint32))


@pytest.mark.parametrize("codes", CODES, ids=lambda c: c[0])
@pytest.mark.parametrize("shape", [(37, 128), (5, 3, 256), (300, 16), (2, 8192), (9, 64)], ids=str)
def test_one_scale_per_element_of_the_last_dimension(port, codes, shape):
    code_dt, zero_dt = codes
    cols = shape[-1]
    rng = np.random.default_rng(cols + len(shape))
    scale = rng.uniform(0.01, 0.05, cols).astype(np.float32)
    scale[3] = 0.0
    zero = (rng.integers(-8, 9, cols) if zero_dt == "int8" else rng.integers(100, 140, cols)).astype(np.int8 if zero_dt == "int8" else np.uint8)
    x = _values(rng, shape, np.where(scale == 0, 1, scale).astype(np.float32))
    for s_arg, z_arg in ((scale, zero), (scale.reshape((1,) * (len(shape) - 1) + (cols,)), zero.reshape((1,) * (len(shape) - 1) + (cols,)))):
        want = port.quantize(x, "float32", s_arg, "float32", z_arg, zero_dt, code_dt, axis=len(shape) - 1)
        got = gpu.quantize(x, "float32", s_arg, "float32", z_arg, zero_dt, code_dt, axis=len(shape) - 1)
        assert _same(got, want), (codes, shape)
    all_codes = rng.integers(0, 256, shape).astype(np.uint8).view(want.dtype)
    s_b, z_b = scale.reshape((1,) * (len(shape) - 1) + (cols,)), zero.reshape((1,) * (len(shape) - 1) + (cols,))
    back_want = port.dequantize(all_codes, code_dt, s_b, "float32", z_b, zero_dt, "float32")
    back = gpu.dequantize(all_codes, code_dt, s_b, "float32", z_b, zero_dt, "float32")
    nan = np.isnan(back_want)
    assert np.array_equal(np.isnan(back), nan) and np.array_equal(back[~nan].view(np.uint32), back_want[~nan].view(np.uint32))


def test_a_square_tensor_quantised_along_its_first_axis_is_not_mistaken_for_the_last(port):
    rng = np.random.default_rng(1)
    x = rng.normal(0, 1, (64, 64)).astype(np.float32)
    scale = rng.uniform(0.01, 0.05, 64).astype(np.float32)
    zero = rng.integers(-8, 9, 64).astype(np.int8)
    want = port.quantize(x, "float32", scale, "float32", zero, "int8", "int8", axis=0)
    got = gpu.quantize(x, "float32", scale, "float32", zero, "int8", "int8", axis=0)
    assert _same(got, want)
    assert not _same(got, port.quantize(x, "float32", scale, "float32", zero, "int8", "int8", axis=1))
