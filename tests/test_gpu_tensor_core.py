"""Tensor-core Gemm / Conv2d against a float64 evaluation of the same low-precision inputs.

The reference accumulates in double; the tensor cores accumulate in float32, so only the order and
width of the accumulation differ.  Gate (per element): |gpu - ref| <= 1e-6 * S + 1 unit in the last
place of the output type, where S = sum_k |a_k * b_k| is the magnitude actually accumulated (never
|y|: cancellation would make a relative-to-result bound meaningless).
"""
import numpy as np
import pytest

import gpu_ops as gpu
from datagen import from_f64, to_f64

pytestmark = pytest.mark.gpu

ULP = {"float32": 2.0 ** -23, "bfloat16": 2.0 ** -7, "float16": 2.0 ** -10}


def _tc_count():
    from onnx_translator_b200 import capi
    return capi.load().tops_tensor_core_launches()


def _gate(got, want, s_mag, out_dt, what):
    tol = 1e-6 * s_mag + ULP[out_dt] * np.abs(want) + 1e-30
    err = np.abs(got - want)
    bad = err > tol
    assert not bad.any(), f"{what}: {int(bad.sum())} of {bad.size} outside the gate, worst ratio {float((err / tol).max()):.3g}"


def _rand(rng, shape, dt, scale):
    if dt in ("float8_e4m3", "float8_e5m2"):
        return from_f64(rng.normal(0, scale, shape), dt)
    return from_f64(rng.normal(0, scale, shape), dt)


GEMM_CASES = [  # M, N, K, a_dt, b_dt, out_dt, bias
    (128, 256, 64, "bfloat16", "bfloat16", "float32", None),
    (256, 512, 1024, "bfloat16", "bfloat16", "float32", "col"),
    (256, 512, 1024, "bfloat16", "bfloat16", "bfloat16", "col"),
    (384, 768, 520, "float16", "float16", "float32", "row"),
    (130, 300, 72, "bfloat16", "bfloat16", "float32", "col"),          # ragged in M, N and K
    (1, 1000, 2048, "float16", "float16", "float16", "scalar"),
    (256, 1000, 2048, "bfloat16", "bfloat16", "float32", "col"),       # the classifier of the ResNet-shaped graph
    (512, 512, 4096, "float8_e4m3", "float8_e4m3", "float32", "col"),
    (200, 260, 144, "float8_e5m2", "float8_e4m3", "bfloat16", "matrix"),
    (2048, 2048, 2048, "bfloat16", "bfloat16", "float32", "col"),
    (1024, 4096, 8192, "bfloat16", "bfloat16", "bfloat16", "col"),     # K of the 8192^3 benchmark case
    (512, 768, 1024, "float32", "float32", "float32", "col"),           # float32 inputs: three-way bfloat16 split
    (1024, 1024, 256, "float32", "float32", "float32", None),
    (640, 520, 2048, "float32", "float32", "bfloat16", "row"),
    (1024, 1024, 128, "bfloat16", "bfloat16", "bfloat16", "col"),      # few K blocks: the variant with eight epilogue warps
    (300, 700, 512, "float16", "float16", "float16", "matrix"),
    (512, 520, 1024, "float8_e4m3", "float8_e5m2", "bfloat16", "row"),
]


@pytest.mark.parametrize("case", GEMM_CASES, ids=lambda c: f"{c[0]}x{c[1]}x{c[2]}-{c[3]}-{c[5]}-{c[6]}")
def test_gemm_tensor_core(case):
    m, n, k, a_dt, b_dt, out_dt, bias_kind = case
    rng = np.random.default_rng(m * 7 + n * 3 + k)
    scale = 0.5 if "float8" in a_dt else 0.02
    a = _rand(rng, (m, k), a_dt, scale)
    b = _rand(rng, (n, k), b_dt, scale)
    bias = {None: None, "col": rng.normal(0, 1, n), "row": rng.normal(0, 1, m), "scalar": rng.normal(0, 1, 1),
            "matrix": rng.normal(0, 1, (m, n))}[bias_kind]
    bias32 = None if bias is None else bias.astype(np.float32)
    alpha, beta = 0.75, 1.25
    before = _tc_count()
    got = to_f64(gpu.gemm(a, a_dt, b, b_dt, bias32, "float32", out_dt, alpha, beta, 0, 1), out_dt)
    assert _tc_count() == before + 1, "the call did not take the tensor-core path"
    a64, b64 = to_f64(a, a_dt), to_f64(b, b_dt)
    want = np.float32(alpha).astype(np.float64) * (a64 @ b64.T)
    if bias32 is not None:
        bb = bias32.astype(np.float64)
        if bias_kind == "row":
            bb = bb.reshape(-1, 1)
        want = want + np.float32(beta).astype(np.float64) * bb
    s_mag = np.abs(a64) @ np.abs(b64).T + (0 if bias32 is None else np.abs(np.broadcast_to(bb, want.shape)) * beta)
    _gate(got, want, s_mag, out_dt, "gemm")


def test_gemm_tensor_core_matches_exact_path_oracle(port):
    """Small case against the C oracle itself (double accumulation in the reference's order)."""
    rng = np.random.default_rng(5)
    a = _rand(rng, (128, 192), "bfloat16", 0.05)
    b = _rand(rng, (256, 192), "bfloat16", 0.05)
    c = rng.normal(0, 1, 256).astype(np.float32)
    got = gpu.gemm(a, "bfloat16", b, "bfloat16", c, "float32", "float32", 1.0, 1.0, 0, 1).astype(np.float64)
    want = port.gemm(a, "bfloat16", b, "bfloat16", c, "float32", "float32", 1.0, 1.0, 0, 1).astype(np.float64)
    s_mag = np.abs(to_f64(a, "bfloat16")) @ np.abs(to_f64(b, "bfloat16")).T + np.abs(c)
    _gate(got, want, s_mag, "float32", "gemm vs oracle")


def test_gemm_unsupported_layouts_fall_back_to_the_exact_kernel(port):
    """transA = 1 is outside the tensor-core path: the exact kernel answers, bit-identical."""
    rng = np.random.default_rng(6)
    a = _rand(rng, (96, 130), "bfloat16", 0.05)       # stored [K, M]
    b = _rand(rng, (260, 96), "bfloat16", 0.05)
    before = _tc_count()
    got = gpu.gemm(a, "bfloat16", b, "bfloat16", None, "float32", "float32", 1.0, 1.0, 1, 1)
    assert _tc_count() == before
    want = port.gemm(a, "bfloat16", b, "bfloat16", None, "float32", "float32", 1.0, 1.0, 1, 1)
    assert np.array_equal(got, want)


# ---- Conv2d ------------------------------------------------------------------------------------------------
def _conv_f64(x, w, b, pads, dil, out_hw):
    """Direct convolution in float64 (stride 1, group 1) and the accumulated magnitude."""
    n, c, h, wd = x.shape
    m, _, kh, kw = w.shape
    oh, ow = out_hw
    xp = np.zeros((n, c, h + pads[0] + pads[2] + kh * dil[0], wd + pads[1] + pads[3] + kw * dil[1]))
    xp[:, :, pads[0]:pads[0] + h, pads[1]:pads[1] + wd] = x
    y = np.zeros((n, m, oh, ow))
    s = np.zeros((n, m, oh, ow))
    for i in range(kh):
        for j in range(kw):
            patch = xp[:, :, i * dil[0]:i * dil[0] + oh, j * dil[1]:j * dil[1] + ow]
            y += np.einsum("nchw,mc->nmhw", patch, w[:, :, i, j], optimize=True)
            s += np.einsum("nchw,mc->nmhw", np.abs(patch), np.abs(w[:, :, i, j]), optimize=True)
    if b is not None:
        y += b.reshape(1, -1, 1, 1)
        s += np.abs(b).reshape(1, -1, 1, 1)
    return y, s


CONV_CASES = [  # N, C, H, W, M, k, pads, dil, x_dt, out_dt, bias
    (4, 64, 28, 28, 128, 3, (1, 1, 1, 1), (1, 1), "bfloat16", "float32", True),
    (2, 256, 56, 56, 256, 3, (1, 1, 1, 1), (1, 1), "bfloat16", "bfloat16", False),     # a slab of the benchmark conv
    (6, 32, 13, 17, 70, 3, (1, 1, 1, 1), (1, 1), "float16", "float16", True),            # odd sizes, ragged channels-out
    (2, 128, 20, 20, 300, 1, (0, 0, 0, 0), (1, 1), "bfloat16", "float32", True),         # 1x1
    (2, 48, 24, 24, 64, 3, (2, 2, 2, 2), (2, 2), "bfloat16", "float32", False),          # dilation 2
    (1, 16, 30, 30, 256, 5, (2, 2, 2, 2), (1, 1), "float16", "float32", True),
    (2, 64, 19, 23, 96, 3, (1, 0, 0, 1), (1, 1), "bfloat16", "float32", True),           # asymmetric padding
    (2, 128, 16, 16, 256, 3, (1, 1, 1, 1), (1, 1), "float8_e4m3", "float32", True),
]


@pytest.mark.parametrize("case", CONV_CASES, ids=lambda c: f"n{c[0]}c{c[1]}h{c[2]}w{c[3]}m{c[4]}k{c[5]}-{c[8]}-{c[9]}")
def test_conv_tensor_core(case):
    n, c, h, wd, m, k, pads, dil, x_dt, out_dt, with_bias = case
    rng = np.random.default_rng(n * 131 + c * 7 + m)
    scale_w = 0.5 if "float8" in x_dt else 0.05
    x = from_f64(rng.normal(0, 1, (n, c, h, wd)), x_dt)
    w = from_f64(rng.normal(0, scale_w, (m, c, k, k)), x_dt)
    b = rng.normal(0, 1, m).astype(np.float32) if with_bias else None
    oh = h + pads[0] + pads[2] - dil[0] * (k - 1)
    ow = wd + pads[1] + pads[3] - dil[1] * (k - 1)
    before = _tc_count()
    got = to_f64(gpu.conv2d(x, x_dt, w, x_dt, b, "float32", out_dt, pads, (1, 1), dil, 1), out_dt)
    assert _tc_count() == before + 1, "the call did not take the tensor-core path"
    want, s_mag = _conv_f64(to_f64(x, x_dt), to_f64(w, x_dt), None if b is None else b.astype(np.float64), pads, dil, (oh, ow))
    assert got.shape == want.shape
    _gate(got, want, s_mag, out_dt, "conv")


def test_conv_tensor_core_against_the_oracle(port):
    rng = np.random.default_rng(77)
    x = from_f64(rng.normal(0, 1, (8, 32, 12, 12)), "bfloat16")
    w = from_f64(rng.normal(0, 0.1, (64, 32, 3, 3)), "bfloat16")
    b = rng.normal(0, 1, 64).astype(np.float32)
    args = (x, "bfloat16", w, "bfloat16", b, "float32", "float32", (1, 1, 1, 1), (1, 1), (1, 1), 1)
    before = _tc_count()
    got = gpu.conv2d(*args).astype(np.float64)
    assert _tc_count() == before + 1
    want = port.conv2d(*args).astype(np.float64)
    _, s_mag = _conv_f64(to_f64(x, "bfloat16"), to_f64(w, "bfloat16"), b.astype(np.float64), (1, 1, 1, 1), (1, 1), (12, 12))
    _gate(got, want, s_mag, "float32", "conv vs oracle")


def test_conv_strided_or_grouped_falls_back_to_the_exact_kernel(port):
    rng = np.random.default_rng(78)
    x = from_f64(rng.normal(0, 1, (2, 32, 16, 16)), "bfloat16")
    w = from_f64(rng.normal(0, 0.1, (64, 32, 3, 3)), "bfloat16")
    args = (x, "bfloat16", w, "bfloat16", None, "float32", "float32", (1, 1, 1, 1), (2, 2), (1, 1), 1)
    before = _tc_count()
    got = gpu.conv2d(*args)
    assert _tc_count() == before
    assert np.array_equal(got, port.conv2d(*args))


# ---- fused DequantizeLinear -> Gemm / Conv -> QuantizeLinear ------------------------------------------------------
@pytest.mark.parametrize("case", [(256, 512, 1024, "float32", "col"), (130, 272, 528, "bfloat16", None), (512, 1024, 2048, "float32", "col")],
                         ids=lambda c: f"{c[0]}x{c[1]}x{c[2]}-{c[3]}")
def test_fused_fp8_gemm_with_operand_scales(port, case):
    """DQ(A), DQ(B) -> Gemm in one call against the same chain evaluated by the oracle in float64."""
    from onnx_translator_b200 import fused
    m, n, k, out_dt, bias_kind = case
    rng = np.random.default_rng(m + n + k)
    sa, sb = np.float32(0.02 / 64), np.float32(0.02 / 48)
    a = from_f64(rng.normal(0, 64, (m, k)), "float8_e4m3")
    b = from_f64(rng.normal(0, 48, (n, k)), "float8_e4m3")
    bias = rng.normal(0, 1, n).astype(np.float32) if bias_kind else None
    zero = np.zeros(1, np.uint8)
    a_dq = port.dequantize(a, "float8_e4m3", np.array([sa]), "float32", zero, "float8_e4m3", "float32").astype(np.float64)
    b_dq = port.dequantize(b, "float8_e4m3", np.array([sb]), "float32", zero, "float8_e4m3", "float32").astype(np.float64)
    want = a_dq @ b_dq.T + (0 if bias is None else bias.astype(np.float64))
    s_mag = np.abs(a_dq) @ np.abs(b_dq).T + (0 if bias is None else np.abs(bias.astype(np.float64)))
    before = _tc_count()
    got = fused.gemm_qdq(a, sa, b, sb, None if bias is None else bias.reshape(1, n), out_dtype=out_dt).numpy()
    assert _tc_count() == before + 1
    _gate(to_f64(got, out_dt), want, s_mag, out_dt, "fused fp8 gemm")


@pytest.mark.parametrize("out_dt", ["float8_e4m3", "float8_e5m2", "int8", "uint8"])
def test_fused_fp8_gemm_quantised_result(port, out_dt):
    """DQ -> Gemm -> Q: every code lies between the codes the oracle's QuantizeLinear gives for the float64 result
    minus and plus the accumulation tolerance -- for each 8-bit result type, with results beyond the type's range
    (saturation for e4m3 and the integers, infinity for e5m2) and a NaN row among them."""
    from onnx_translator_b200 import fused
    m, n, k = 384, 512, 1024
    rng = np.random.default_rng(5)
    sa, sb = np.float32(1 / 1024), np.float32(1 / 2048)
    sy = np.float32({"float8_e4m3": 1 / 16, "float8_e5m2": 1 / 4096, "int8": 1 / 8, "uint8": 1 / 8}[out_dt])
    a = from_f64(rng.normal(0, 40, (m, k)), "float8_e4m3")
    b = from_f64(rng.normal(0, 90, (n, k)), "float8_e4m3")
    a[7, :] = 0x7F                                                    # a NaN operand row: the whole result row is NaN
    bias = rng.normal(0, 1, n).astype(np.float32)
    bias[::37] = 1e9 if out_dt != "float8_e5m2" else 3e4             # far beyond the range / past e5m2's overflow threshold after scaling
    bias[5::41] = -1e9 if out_dt != "float8_e5m2" else -3e4
    zero_dt = out_dt if out_dt in ("int8", "uint8") else "float8_e4m3"
    zero = np.zeros(1, np.int8 if zero_dt == "int8" else np.uint8)
    e4_zero = np.zeros(1, np.uint8)
    a_dq = port.dequantize(a, "float8_e4m3", np.array([sa]), "float32", e4_zero, "float8_e4m3", "float32").astype(np.float64)
    b_dq = port.dequantize(b, "float8_e4m3", np.array([sb]), "float32", e4_zero, "float8_e4m3", "float32").astype(np.float64)
    with np.errstate(invalid="ignore"):
        y = a_dq @ b_dq.T + bias.astype(np.float64)
        tol = 1e-6 * (np.abs(a_dq) @ np.abs(b_dq).T + np.abs(bias)) + 2.0 ** -23 * np.abs(y)
    finite = np.isfinite(y)
    lo = np.nextafter(np.where(finite, y - tol, 0).astype(np.float32), np.float32(-np.inf))
    hi = np.nextafter(np.where(finite, y + tol, 0).astype(np.float32), np.float32(np.inf))
    q = lambda v: to_f64(port.quantize(v, "float32", np.array([sy]), "float32", zero, zero_dt, out_dt), out_dt)
    q_lo, q_hi = q(lo), q(hi)
    got_codes = fused.gemm_qdq(a, sa, b, sb, bias.reshape(1, n), y_scale=sy, out_dtype=out_dt).numpy()
    got = to_f64(got_codes, out_dt)
    inside = (got >= q_lo) & (got <= q_hi)
    assert np.all(inside[finite]), int((~inside[finite]).sum())
    want_nan_row = port.quantize(np.full(n, np.nan, np.float32), "float32", np.array([sy]), "float32", zero, zero_dt, out_dt)
    if out_dt in ("int8", "uint8"):
        assert np.array_equal(got_codes[7], want_nan_row)            # the x86 float -> integer conversion of NaN: the most negative value
    else:
        assert np.all(np.isnan(got[7]))
    rows = np.arange(m) != 7
    assert np.mean(got[rows] == q(y.astype(np.float32))[rows]) > 0.999
    assert np.unique(got[rows]).size > 20                             # a real spread of codes, not a saturated output
    if out_dt == "float8_e5m2":
        assert np.isinf(got[rows][:, ::37]).all() and np.isinf(got[rows][:, 5::41]).all()


@pytest.mark.parametrize("x_dt", ["bfloat16", "float16"])
def test_fused_conv_with_int8_weights(port, x_dt):
    """DQ(W per output channel) -> Conv in one call against the chain in float64."""
    from onnx_translator_b200 import fused
    rng = np.random.default_rng(91)
    n, c, h, wd, m = 4, 64, 28, 28, 96
    x = from_f64(rng.normal(0, 1, (n, c, h, wd)), x_dt)
    wq = rng.integers(-127, 128, (m, c, 3, 3)).astype(np.int8)
    ws = rng.uniform(0.005, 0.02, m).astype(np.float32)
    b = rng.normal(0, 1, m).astype(np.float32)
    full_scale = np.ascontiguousarray(np.broadcast_to(ws.reshape(m, 1, 1, 1), wq.shape))
    w_dq = port.dequantize(wq, "int8", full_scale, "float32", np.zeros(wq.shape, np.int8), "int8", "float32").astype(np.float64)
    want, s_mag = _conv_f64(to_f64(x, x_dt), w_dq, b.astype(np.float64), (1, 1, 1, 1), (1, 1), (h, wd))
    before = _tc_count()
    got = fused.conv2d_dqw(x, wq, ws, b, out_dtype="float32", pads=(1, 1, 1, 1), x_dtype=x_dt).numpy().astype(np.float64)
    assert _tc_count() == before + 1
    _gate(got, want, s_mag, "float32", "fused conv with int8 weights")


def test_fused_entry_points_refuse_what_they_do_not_cover():
    from onnx_translator_b200 import capi, fused
    rng = np.random.default_rng(3)
    a = from_f64(rng.normal(0, 1, (64, 64)), "bfloat16")
    with pytest.raises(capi.TensorOpsError):
        fused.gemm_qdq(a, 1.0, a, 1.0, a_dtype="bfloat16", b_dtype="bfloat16")          # not fp8
    x = rng.normal(0, 1, (1, 16, 8, 8)).astype(np.float32)
    with pytest.raises(capi.TensorOpsError):
        fused.conv2d_dqw(x, np.ones((16, 16, 3, 3), np.int8), np.ones(16, np.float32), x_dtype="float32")   # float32 activations


QCONV_CASES = [  # N, C, H, W, M, k, pad, stride, x_dt, zero, relu, bias
    (4, 64, 28, 28, 96, 3, 1, 1, "int8", 0, True, True),
    (2, 3, 64, 64, 64, 7, 3, 2, "int8", 0, True, True),          # the stem: 7x7 stride 2 on 3 channels
    (3, 32, 30, 30, 70, 3, 1, 2, "int8", 5, False, True),        # 3x3 stride 2, non-zero zero point
    (2, 64, 28, 28, 128, 1, 0, 2, "int8", 0, False, False),      # the 1x1 stride-2 shortcut
    (2, 20, 17, 19, 40, 1, 0, 1, "uint8", 128, True, True),      # channels not a multiple of 8, odd sizes
    (2, 24, 15, 15, 48, 3, 1, 2, "uint8", 100, True, False),     # odd extent with stride 2
    (1, 256, 14, 14, 512, 3, 1, 1, "int8", -3, False, True),
    (2, 3, 20, 22, 32, 3, 1, 1, "int8", 0, True, True),            # few channels: the taps of a filter row share a K block
    (2, 16, 20, 20, 40, 3, 1, 1, "uint8", 7, False, True),
    (3, 8, 18, 18, 24, 5, 2, 1, "int8", 1, True, False),
    (2, 5, 33, 31, 16, 7, 3, 2, "int8", -4, True, True),
    (2, 1, 21, 23, 16, 3, 1, 2, "uint8", 9, True, True),           # one channel (its own instance of the per-cell layout kernel)
    (2, 4, 18, 18, 24, 3, 1, 1, "int8", -2, False, True),          # four channels (likewise)
    (1, 2, 16, 20, 16, 5, 2, 2, "int8", 3, True, False),           # two channels, stride 2: the generic instance
]


@pytest.mark.parametrize("case", QCONV_CASES, ids=lambda c: f"n{c[0]}c{c[1]}h{c[2]}m{c[4]}k{c[5]}s{c[7]}-{c[8]}z{c[9]}")
def test_qlinear_conv_against_the_unfused_chain_in_float64(port, case):
    """DQ(x codes) + DQ(w codes) + Conv [+ Relu] in one call against the oracle's DequantizeLinear outputs
    convolved in float64, gated on the accumulated magnitude."""
    from onnx_translator_b200.nn import Tensor
    from onnx_translator_b200.nn.fused_ops import QLinearConv
    n, c, h, wd, m, k, pad, stride, x_dt, zero, relu, with_bias = case
    rng = np.random.default_rng(n * 1000 + c * 10 + k + stride)
    lo, hi = (-128, 128) if x_dt == "int8" else (0, 256)
    xq = rng.integers(lo, hi, (n, c, h, wd)).astype(np.int8 if x_dt == "int8" else np.uint8)
    wq = rng.integers(-127, 128, (m, c, k, k)).astype(np.int8)
    sx = np.array([0.037], np.float32)
    zx = np.array([zero], xq.dtype)
    ws = rng.uniform(0.005, 0.02, (m, 1, 1, 1)).astype(np.float32)
    b = rng.normal(0, 1, m).astype(np.float32) if with_bias else None
    x_dq = port.dequantize(xq, x_dt, sx, "float32", zx, x_dt, "float32").astype(np.float64)
    w_dq = port.dequantize(wq, "int8", ws, "float32", np.zeros((m, 1, 1, 1), np.int8), "int8", "float32").astype(np.float64)
    oh1, ow1 = h + 2 * pad - (k - 1), wd + 2 * pad - (k - 1)
    full, s_full = _conv_f64(x_dq, w_dq, None if b is None else b.astype(np.float64), (pad,) * 4, (1, 1), (oh1, ow1))
    want, s_mag = full[:, :, ::stride, ::stride], s_full[:, :, ::stride, ::stride]
    if relu:
        want = np.maximum(want, 0)
    node = QLinearConv([], [], [pad] * 4, [stride, stride], [1, 1], relu, "float32")
    T = lambda a, dt: Tensor(*a.shape, dtype=dt, data=a)
    before = _tc_count()
    got = node.forward(T(xq, x_dt), T(sx, "float32"), T(zx, x_dt), T(wq, "int8"), T(ws, "float32"),
                       None if b is None else T(b, "float32"))["tensor"].numpy().astype(np.float64)
    assert _tc_count() == before + 1
    assert got.shape == want.shape
    _gate(got, want, s_mag, "float32", "qlinear conv")
    # one operator earlier: float32 activations whose QuantizeLinear codes are exactly xq (values at and
    # around the rounding ties and beyond the saturation limits included) must give the same bits
    x = ((xq.astype(np.float64) - zero) * sx[0]).astype(np.float32)
    x.reshape(-1)[::7] += np.float32(0.3 * sx[0])
    x.reshape(-1)[3::11] -= np.float32(0.49 * sx[0])
    x.reshape(-1)[5::13] = np.float32(1e6)
    x.reshape(-1)[6::17] = np.nextafter((xq.reshape(-1)[6::17].astype(np.float64) - zero + 0.5) * sx[0], np.inf).astype(np.float32)
    codes = port.quantize(x, "float32", sx, "float32", zx, x_dt, x_dt)
    from_codes = node.forward(T(codes, x_dt), T(sx, "float32"), T(zx, x_dt), T(wq, "int8"), T(ws, "float32"),
                              None if b is None else T(b, "float32"))["tensor"].numpy()
    node_f = QLinearConv([], [], [pad] * 4, [stride, stride], [1, 1], relu, "float32", from_float=True)
    from_float = node_f.forward(T(x, "float32"), T(sx, "float32"), T(zx, x_dt), T(wq, "int8"), T(ws, "float32"),
                                None if b is None else T(b, "float32"))["tensor"].numpy()
    assert np.array_equal(from_codes.view(np.uint32), from_float.view(np.uint32))


def test_qlinear_conv_with_residual_equals_the_three_operators_bit_for_bit():
    """Conv + Add(residual) + Relu in the epilogue rounds exactly like the three float32 operators in sequence."""
    from onnx_translator_b200.nn import Tensor
    from onnx_translator_b200.nn import Operators as ops
    from onnx_translator_b200.nn.fused_ops import QLinearConv
    rng = np.random.default_rng(8)
    n, c, h, m = 3, 32, 20, 72
    x = rng.normal(0, 1, (n, c, h, h)).astype(np.float32)
    wq = rng.integers(-127, 128, (m, c, 3, 3)).astype(np.int8)
    sx, zx = np.array([0.03], np.float32), np.array([2], np.int8)
    ws = rng.uniform(0.005, 0.02, (m, 1, 1, 1)).astype(np.float32)
    b = rng.normal(0, 1, m).astype(np.float32)
    res = rng.normal(0, 3, (n, m, h, h)).astype(np.float32)
    T = lambda a, dt: Tensor(*a.shape, dtype=dt, data=a)
    args = (T(x, "float32"), T(sx, "float32"), T(zx, "int8"), T(wq, "int8"), T(ws, "float32"), T(b, "float32"))
    plain = QLinearConv([], [], [1] * 4, [1, 1], [1, 1], False, "float32", from_float=True).forward(*args)["tensor"]
    want = ops.RELU([], [], dtype="float32").forward(ops.ADD([], [], dtype="float32").forward(plain, T(res, "float32"))["tensor"])["tensor"].numpy()
    got = QLinearConv([], [], [1] * 4, [1, 1], [1, 1], True, "float32", from_float=True).forward(*args, T(res, "float32"))["tensor"].numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))
    no_relu = QLinearConv([], [], [1] * 4, [1, 1], [1, 1], False, "float32", from_float=True).forward(*args, T(res, "float32"))["tensor"].numpy()
    want2 = ops.ADD([], [], dtype="float32").forward(plain, T(res, "float32"))["tensor"].numpy()
    assert np.array_equal(no_relu.view(np.uint32), want2.view(np.uint32))


@pytest.mark.parametrize("nxt", [(3, 1, 1, "int8", 0), (3, 2, 1, "int8", 4), (1, 1, 0, "uint8", 128), (1, 2, 0, "int8", -2), (5, 1, 2, "uint8", 17)],
                         ids=lambda c: f"next-k{c[0]}s{c[1]}p{c[2]}-{c[3]}z{c[4]}")
def test_levels_edge_between_two_quantised_convolutions_is_bit_identical(nxt):
    """conv A -> (integer levels in B's layout) -> conv B must equal conv A -> float32 -> Q -> conv B bit for bit:
    the epilogue of A quantises with the arithmetic of QuantizeLinear and writes B's padded / space-to-depth layout."""
    from onnx_translator_b200.nn import Tensor
    from onnx_translator_b200.nn.fused_ops import QLinearConv
    k2, s2, p2, code_dt, zero2 = nxt
    rng = np.random.default_rng(k2 * 10 + s2)
    n, c, h, m1, m2 = 3, 16, 22, 40, 24
    T = lambda a, dt: Tensor(*a.shape, dtype=dt, data=a)
    x = T(rng.normal(0, 1, (n, c, h, h)).astype(np.float32), "float32")
    sx, zx = T(np.array([0.03], np.float32), "float32"), T(np.zeros(1, np.int8), "int8")
    w1 = T(rng.integers(-127, 128, (m1, c, 3, 3)).astype(np.int8), "int8")
    w1s = T(rng.uniform(0.002, 0.01, (m1, 1, 1, 1)).astype(np.float32), "float32")
    b1 = T(rng.normal(0, 0.5, m1).astype(np.float32), "float32")
    res = T(rng.normal(0, 1, (n, m1, h, h)).astype(np.float32), "float32")
    s2t = T(np.array([0.05], np.float32), "float32")
    z2t = T(np.array([zero2], np.int8 if code_dt == "int8" else np.uint8), code_dt)
    w2 = T(rng.integers(-127, 128, (m2, m1, k2, k2)).astype(np.int8), "int8")
    w2s = T(rng.uniform(0.002, 0.01, (m2, 1, 1, 1)).astype(np.float32), "float32")

    def conv_a(next_conv):
        node = QLinearConv([], [], [1] * 4, [1, 1], [1, 1], True, "float32", from_float=True)
        node.next_conv = next_conv
        return node.forward(x, sx, zx, w1, w1s, b1, res, *((s2t, z2t) if next_conv else ()))["tensor"]

    def conv_b(inp, levels_in):
        node = QLinearConv([], [], [p2] * 4, [s2, s2], [1, 1], False, "float32", from_float=True)
        node.levels_in = levels_in
        return node.forward(inp, s2t, z2t, w2, w2s)["tensor"].numpy()

    want = conv_b(conv_a(None), False)
    levels = conv_a(dict(pads=[p2] * 4, strides=[s2, s2], dilations=[1, 1], kernel=[k2, k2]))
    assert levels.dtype == "bfloat16" and levels.logical_shape == (n, m1, h, h)
    got = conv_b(levels, True)
    assert got.shape == want.shape and np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_filter_cache_is_reused_and_follows_the_weight_array():
    """The node keeps the filters in tensor-core layout between calls: a second call gives identical bytes, and a
    different weight array (not the stale cache) decides the result of the third."""
    from onnx_translator_b200.nn import Tensor
    from onnx_translator_b200.nn.fused_ops import QLinearConv
    rng = np.random.default_rng(321)
    T = lambda a, dt: Tensor(*a.shape, dtype=dt, data=a)
    x = T(rng.normal(0, 1, (2, 32, 14, 14)).astype(np.float32), "float32")
    sx, zx = T(np.array([0.04], np.float32), "float32"), T(np.zeros(1, np.int8), "int8")
    w1 = T(rng.integers(-127, 128, (48, 32, 3, 3)).astype(np.int8), "int8")
    w2 = T(rng.integers(-127, 128, (48, 32, 3, 3)).astype(np.int8), "int8")
    ws = T(rng.uniform(0.002, 0.01, (48, 1, 1, 1)).astype(np.float32), "float32")
    node = QLinearConv([], [], [1] * 4, [1, 1], [1, 1], True, "float32", from_float=True)
    fresh = lambda w: QLinearConv([], [], [1] * 4, [1, 1], [1, 1], True, "float32", from_float=True).forward(x, sx, zx, w, ws)["tensor"].numpy()
    first = node.forward(x, sx, zx, w1, ws)["tensor"].numpy()
    assert node._filter_cache.value
    kept = node._filter_cache.value
    second = node.forward(x, sx, zx, w1, ws)["tensor"].numpy()
    assert node._filter_cache.value == kept and np.array_equal(first, second) and np.array_equal(first, fresh(w1))
    third = node.forward(x, sx, zx, w2, ws)["tensor"].numpy()
    assert np.array_equal(third, fresh(w2)) and not np.array_equal(third, first)
