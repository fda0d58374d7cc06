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
