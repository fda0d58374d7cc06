"""MatMul and DynamicQuantizeLinear on the GPU.

MatMul on the exact path (every dtype combination the tensor cores do not take) is bit-identical to the oracle; on
the tensor-core path (float16 / bfloat16 / fp8 pairs, large float32 problems) the gate is that of Gemm: float32
accumulation of exact products, |err| <= 1e-6 * sum|a||b| + one unit in the last place of the output type.
DynamicQuantizeLinear is bit-identical: codes, scale and zero point."""
import zlib

import numpy as np
import pytest

import gpu_ops as gpu
from datagen import assert_same_codes, from_f64, make, to_f64

pytestmark = pytest.mark.gpu

ULP = {"float32": 2.0 ** -23, "bfloat16": 2.0 ** -7, "float16": 2.0 ** -10}


def _tc_count():
    from onnx_translator_b200 import capi
    return capi.load().tops_tensor_core_launches()


EXACT_PLANS = [  # a_dt, b_dt, out_dt, a shape, b shape
    ("float32", "float32", "float32", (7, 13), (13, 5)),
    ("float32", "float32", "float32", (3, 2, 70, 130), (130, 50)),            # batched A, one B: a single tall problem
    ("float32", "float32", "float32", (4, 6, 9), (4, 9, 11)),                  # equal batches
    ("bfloat16", "float32", "float32", (2, 1, 6, 8), (1, 3, 8, 4)),            # mixed broadcasting
    ("float64", "float64", "float64", (5, 17), (2, 17, 3)),                    # one A, batched B
    ("int8", "int8", "int32", (3, 5, 12), (12, 7)),
    ("int32", "float32", "float64", (1, 4, 6), (5, 6, 2)),
    ("float16", "float16", "float16", (4, 6, 9), (4, 9, 11)),                  # K * 2 bytes not a multiple of 16: exact kernel
    ("float32", "float32", "int8", (1, 9), (9, 1)),
    ("float32", "float32", "float32", (2, 3, 65, 0), (0, 70)),                 # empty inner dimension: zeros
    ("float32", "float32", "float16", (200, 3, 33), (200, 33, 65)),
]


@pytest.mark.parametrize("plan", EXACT_PLANS, ids=lambda p: f"{p[0]}-{p[1]}-{p[2]}-{'x'.join(map(str, p[3]))}@{'x'.join(map(str, p[4]))}")
def test_matmul_exact_path_is_bit_identical(port, plan):
    a_dt, b_dt, out_dt, a_shape, b_shape = plan
    rng = np.random.default_rng(zlib.crc32(repr(plan).encode()))
    a, b = make(rng, a_shape, a_dt), make(rng, b_shape, b_dt)
    before = _tc_count()
    got = gpu.matmul(a, a_dt, b, b_dt, out_dt)
    assert _tc_count() == before
    assert_same_codes(got, port.matmul(a, a_dt, b, b_dt, out_dt), out_dt, repr(plan))


def test_matmul_promotes_one_dimensional_operands(port):
    rng = np.random.default_rng(5)
    v, m, w = make(rng, (12,), "float32"), make(rng, (3, 12, 8), "float32"), make(rng, (8,), "float32")
    got = gpu.matmul(v, "float32", m, "float32", "float32")
    assert got.shape == (3, 8)
    assert_same_codes(got, port.matmul(v.reshape(1, 12), "float32", m, "float32", "float32").reshape(3, 8), "float32")
    got = gpu.matmul(m, "float32", w, "float32", "float32")
    assert got.shape == (3, 12)
    assert_same_codes(got, port.matmul(m, "float32", w.reshape(8, 1), "float32", "float32").reshape(3, 12), "float32")
    got = gpu.matmul(v, "float32", v, "float32", "float32")
    assert got.shape == ()
    with pytest.raises(ValueError):
        gpu.matmul(v, "float32", w, "float32", "float32")
    with pytest.raises(ValueError):
        gpu.matmul(make(rng, (2, 3, 4), "float32"), "float32", make(rng, (3, 4, 5), "float32"), "float32", "float32")


TC_PLANS = [  # a_dt, out_dt, a shape, b shape, tensor-core launches expected
    ("bfloat16", "float32", (256, 512), (512, 384), 1),
    ("float16", "float16", (4, 8, 128, 64), (64, 256), 1),                      # collapsed to 4096 rows
    ("bfloat16", "bfloat16", (6, 130, 72), (6, 72, 200), 1),                     # equal batches: one launch, ragged tiles
    ("float16", "float32", (2, 5, 300, 64), (2, 5, 64, 136), 1),
    ("float8_e5m2", "float16", (3, 64, 128), (3, 128, 96), 1),
    ("float8_e4m3", "float32", (2, 3, 64, 128), (1, 3, 128, 96), 6),
    ("bfloat16", "float32", (2, 1, 64, 64), (1, 3, 64, 128), 6),                 # mixed broadcasting
    ("float32", "float32", (2, 512, 1024), (2, 1024, 768), 2),                   # float32: three-way bfloat16 split
]


@pytest.mark.parametrize("plan", TC_PLANS, ids=lambda p: f"{p[0]}-{p[1]}-{'x'.join(map(str, p[2]))}@{'x'.join(map(str, p[3]))}")
def test_matmul_tensor_core_path(plan):
    dt, out_dt, a_shape, b_shape, launches = plan
    rng = np.random.default_rng(zlib.crc32(repr(plan).encode()))
    scale = 0.5 if "float8" in dt else 0.05
    a, b = from_f64(rng.normal(0, scale, a_shape), dt), from_f64(rng.normal(0, scale, b_shape), dt)
    before = _tc_count()
    got = to_f64(gpu.matmul(a, dt, b, dt, out_dt), out_dt)
    assert _tc_count() == before + launches
    a64, b64 = to_f64(a, dt), to_f64(b, dt)
    want, mag = np.matmul(a64, b64), np.matmul(np.abs(a64), np.abs(b64))
    err, tol = np.abs(got - want), 1e-6 * mag + ULP[out_dt] * np.abs(want) + 1e-30
    assert (err <= tol).all(), f"worst ratio {float((err / tol).max()):.3g}"


@pytest.mark.parametrize("x_dt", ["float32", "float16", "bfloat16", "float64", "int8", "float8_e5m2"])
def test_dynamic_quantize_linear_is_bit_identical(port, x_dt):
    rng = np.random.default_rng(zlib.crc32(x_dt.encode()))
    cases = [make(rng, (5, 77), x_dt), make(rng, (3, 64, 56, 56), x_dt, -1.5, 4.0) if x_dt != "int8" else make(rng, (3, 64, 56, 56), x_dt),
             from_f64(np.abs(rng.normal(0, 2, 4099)), x_dt), from_f64(-np.abs(rng.normal(0, 2, 333)), x_dt),
             from_f64(np.zeros((4, 4)), x_dt), from_f64(np.full((3,), 2.5), x_dt), from_f64(np.zeros((0,)), x_dt)]
    if x_dt == "float32":
        odd = make(rng, (64,), x_dt)
        odd[:3] = [np.nan, 1e30, -3.0]
        cases.append(odd)
        inf = make(rng, (16,), x_dt)
        inf[2], inf[5] = -np.inf, np.inf
        cases.append(inf)
        halves = (np.arange(-40, 41) * 0.5 * (10.0 / 255.0)).astype(np.float32)        # quotients at and near .5 ties
        cases.append(np.concatenate([halves, np.float32([-5.0, 5.0])]))
        cases.append(make(rng, (1 << 22,), x_dt)[1:])                                   # a view that is not 16-byte aligned on the host
    for x in cases:
        got, want = gpu.dynamic_quantize_linear(x, x_dt), port.dynamic_quantize_linear(x, x_dt)
        for g, w, dt, what in zip(got, want, ("uint8", "float32", "uint8"), ("codes", "scale", "zero point")):
            assert_same_codes(g, w, dt, f"{x_dt} {x.shape} {what}")


def test_dynamic_quantize_linear_large_tensor_properties():
    """At a size the oracle does not finish quickly: the codes reproduce x within half a step, 0 maps onto the zero point."""
    rng = np.random.default_rng(11)
    x = rng.normal(0.3, 1.0, (64, 1 << 20)).astype(np.float32)
    x[3, 17] = 0.0
    y, scale, zero = gpu.dynamic_quantize_linear(x, "float32")
    lo, hi = min(float(x.min()), 0.0), max(float(x.max()), 0.0)
    assert scale[0] == np.float32((hi - lo) / 255.0)
    assert zero[0] == int(np.clip(np.floor(-lo / ((hi - lo) / 255.0) + 0.5), 0, 255))
    assert y[3, 17] == zero[0] and y.min() == 0 and y.max() == 255
    back = (y.astype(np.float64) - float(zero[0])) * ((hi - lo) / 255.0)
    assert np.abs(back - x).max() <= 0.5 * (hi - lo) / 255.0 * (1 + 1e-6) + abs(lo / ((hi - lo) / 255.0) + float(zero[0])) * (hi - lo) / 255.0


@pytest.mark.parametrize("x_dt", ["float32", "float16", "int32"])
def test_dynamic_quantize_range_and_apply_equal_the_single_call(port, x_dt):
    """The split entry points used when the rows of a tensor live on several GPUs: on one GPU, two row blocks
    with their ranges combined on the host must give the codes, scale and zero point of the single call."""
    import ctypes
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    rng = np.random.default_rng(zlib.crc32(x_dt.encode()) + 1)
    x = make(rng, (37, 1000), x_dt)
    if x_dt == "float32":
        x[3, 5], x[30, 7] = np.nan, np.nan
    want = port.dynamic_quantize_linear(x, x_dt)
    blocks = [DeviceArray.from_numpy(np.ascontiguousarray(b), x_dt) for b in (x[:20], x[20:])]
    ranges = [DeviceArray.empty((2,), "float64") for _ in blocks]
    for b, r in zip(blocks, ranges):
        assert lib.tops_dynamic_quantize_range(b.handle, r.handle) == 0
    host = [r.numpy() for r in ranges]
    for h, b in zip(host, (x[:20], x[20:])):
        assert np.array_equal(h, port.dynamic_quantize_range(b, x_dt))
    common = DeviceArray.from_numpy(np.array([min(host[0][0], host[1][0]), max(host[0][1], host[1][1])]), "float64")
    codes = []
    for b in blocks:
        y, s, z = DeviceArray.empty(b.shape, "uint8"), DeviceArray.empty((1,), "float32"), DeviceArray.empty((1,), "uint8")
        assert lib.tops_dynamic_quantize_apply(b.handle, common.handle, y.handle, s.handle, z.handle) == 0
        codes.append(y.numpy())
        assert_same_codes(s.numpy(), want[1], "float32")
        assert_same_codes(z.numpy(), want[2], "uint8")
    assert_same_codes(np.concatenate(codes), want[0], "uint8")
    bad = DeviceArray.empty((2,), "float32")
    assert lib.tops_dynamic_quantize_range(blocks[0].handle, bad.handle) != 0
    lib.tops_clear_error()
