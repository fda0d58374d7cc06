"""Q/DQ fused with elementwise neighbours (tops_quantize_dequantize_forward, tops_dq_add_q_forward) against the
oracle evaluating the separate operators (tensor_ops.c:999-1034, 864-997, 708-728): bit for bit."""
import numpy as np
import pytest

from datagen import from_f64

pytestmark = pytest.mark.gpu


def _t(a, dt):
    from onnx_translator_b200 import nn
    a = np.asarray(a)
    return nn.Tensor(*a.shape, dtype=dt, data=a)


def _same(got, want):
    return got.shape == want.shape and np.array_equal(np.ascontiguousarray(got).view(np.uint8), np.ascontiguousarray(want).view(np.uint8))


ROUND_TRIPS = [  # code dtype, zero dtype, scale kind, zero value(s)
    ("int8", "int8", "tensor", 0),
    ("uint8", "uint8", "tensor", 128),
    ("int8", "int8", "axis", None),
    ("float8_e4m3", "int8", "tensor", 0),
    ("float8_e5m2", "int8", "tensor", 0),
    ("float8_e4m3", "float8_e4m3", "tensor", 0),
]


@pytest.mark.parametrize("case", ROUND_TRIPS, ids=lambda c: f"{c[0]}-z{c[1]}-{c[2]}")
@pytest.mark.parametrize("shape", [(64, 256), (7, 33), (3, 16, 5, 9)], ids=str)
def test_quantize_dequantize_round_trip_equals_the_two_operators(port, case, shape):
    from onnx_translator_b200.nn.fused_ops import QuantizeDequantize
    code_dt, zero_dt, kind, zero = case
    rng = np.random.default_rng(len(shape) * 100 + shape[-1])
    x = rng.normal(0, 1, shape).astype(np.float32)
    flat = x.reshape(-1)
    flat[::5] = (np.rint(flat[::5] / 0.02) + 0.5).astype(np.float32) * np.float32(0.02)      # at and next to rounding ties
    flat[1::7] *= 300                                                                       # beyond the saturation limits
    flat[2::31] = np.float32(1e30)
    axis = 1
    if kind == "axis":
        c = shape[axis]
        scale = rng.uniform(0.01, 0.05, c).astype(np.float32)
        zp = rng.integers(-8, 9, c).astype(np.int8)
        bshape = [1] * len(shape)
        bshape[axis] = c
        s_b, z_b = scale.reshape(bshape), zp.reshape(bshape)
    else:
        scale = np.array([0.02 if "float8" not in code_dt else 1 / 16], np.float32)
        zp = from_f64(np.array([float(zero)]), zero_dt) if "float8" in zero_dt else np.array([zero], np.int8 if zero_dt == "int8" else np.uint8)
        s_b, z_b = scale, zp
    want_codes = port.quantize(x, "float32", s_b, "float32", z_b, zero_dt, code_dt)
    want = port.dequantize(want_codes, code_dt, s_b, "float32", z_b, zero_dt, "float32")
    for with_codes in (False, True):
        if not with_codes and code_dt != zero_dt:
            continue                    # without a codes tensor the code type is the zero point's type
        node = QuantizeDequantize([], [], axis=axis, code_dtype=code_dt, with_codes=with_codes)
        res = node.forward(_t(x, "float32"), _t(scale, "float32"), _t(zp, zero_dt))["tensor"]
        y, codes = res if with_codes else (res, None)
        assert _same(y.numpy(), want), (case, shape, with_codes)
        if with_codes:
            assert _same(codes.numpy(), want_codes)


@pytest.mark.parametrize("dts", [("int8", "int8", "int8"), ("int8", "uint8", "int8"), ("uint8", "uint8", "uint8"), ("uint8", "int8", "uint8")], ids="-".join)
@pytest.mark.parametrize("relu", [False, True])
@pytest.mark.parametrize("shape", [(4, 32, 14, 14), (3, 5, 7)], ids=str)
def test_dequantize_add_quantize_equals_the_chain(port, dts, relu, shape):
    from onnx_translator_b200.nn.fused_ops import DequantAddQuant
    da, db, dy = dts
    rng = np.random.default_rng(sum(map(len, dts)) * 10 + int(relu) + len(shape))
    npdt = lambda d: np.int8 if d == "int8" else np.uint8
    draw = lambda d: rng.integers(-128 if d == "int8" else 0, 128 if d == "int8" else 256, shape).astype(npdt(d))
    a, b = draw(da), draw(db)
    sa, sb, sy = (np.array([v], np.float32) for v in (0.05, 0.021, 0.043))
    za = np.array([3 if da == "int8" else 120], npdt(da))
    zb = np.array([-7 if db == "int8" else 131], npdt(db))
    zy = np.array([-5 if dy == "int8" else 10], npdt(dy))
    f32 = "float32"
    t = port.binary("add", port.dequantize(a, da, sa, f32, za, da, f32), f32, port.dequantize(b, db, sb, f32, zb, db, f32), f32, f32)
    if relu:
        t = port.unary("relu", t, f32, f32)
    want = port.quantize(t, f32, sy, f32, zy, dy, dy)
    got = DequantAddQuant([], [], relu=relu, dtype=dy).forward(_t(a, da), _t(sa, f32), _t(za, da), _t(b, db), _t(sb, f32), _t(zb, db),
                                                                 _t(sy, f32), _t(zy, dy))["tensor"].numpy()
    assert _same(got, want)
    assert np.unique(got).size > 20


def test_fused_elementwise_graph_equals_the_unfused_graph():
    from test_graph import _hand_built_quantised_add
    from onnx_translator_b200 import nn
    rng = np.random.default_rng(11)
    shape = (2, 24, 10, 10)
    a = nn.Tensor(*shape, dtype="int8", data=rng.integers(-128, 128, shape).astype(np.int8))
    b = nn.Tensor(*shape, dtype="uint8", data=rng.integers(0, 256, shape).astype(np.uint8))
    x = nn.Tensor(*shape, dtype="float32", data=rng.normal(0, 2, shape).astype(np.float32))
    graph = _hand_built_quantised_add()
    want = [t.numpy() for t in graph.forward(a, b, x)]
    fused = graph.fused()
    assert [type(op).__name__ for op in fused.ops.values()] == ["DequantAddQuant", "DequantizeLinear", "QuantizeDequantize"]
    got = [t.numpy() for t in fused.forward(a, b, x)]
    assert all(_same(g, w) for g, w in zip(got, want))


def test_fused_calls_refuse_what_they_do_not_cover():
    from onnx_translator_b200 import capi
    from onnx_translator_b200.device import DeviceArray
    lib = capi.load()
    x = DeviceArray.from_numpy(np.ones((4, 4), np.float16), "float16")
    s = DeviceArray.from_numpy(np.array([0.1], np.float32), "float32")
    z = DeviceArray.from_numpy(np.zeros(1, np.int8), "int8")
    y = DeviceArray.from_numpy(np.ones((4, 4), np.float32), "float32")
    assert lib.tops_quantize_dequantize_forward(x.handle, s.handle, z.handle, None, y.handle) == 5
    lib.tops_clear_error()
    assert not y.numpy().any()                          # refused calls leave a zero-filled output
    a = DeviceArray.from_numpy(np.ones((4, 4), np.int8), "int8")
    b = DeviceArray.from_numpy(np.ones((1, 4), np.int8), "int8")
    yq = DeviceArray.from_numpy(np.ones((4, 4), np.int8), "int8")
    assert lib.tops_dq_add_q_forward(a.handle, s.handle, z.handle, b.handle, s.handle, z.handle, s.handle, z.handle, yq.handle, 0) == 5
    lib.tops_clear_error()
