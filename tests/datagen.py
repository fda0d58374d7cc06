"""Seeded input generators shared by the tests.

Value distributions follow the reference's own harness (numerical_correctness.py:110-138):
integers uniform in a range that keeps results representable, fp8 as uniformly random bit
patterns (so NaN/Inf/subnormal codes appear), other floats as a 50/25/25 % mixture of
U(-10,10), U(-1000,1000) and U(-0.01,0.01).  Arrays use the reference's storage convention:
fp8 -> uint8 codes, bfloat16 -> uint16 codes, int4 -> int8.
"""
from __future__ import annotations

import numpy as np

FLOAT_DTYPES = ("float8_e4m3", "float8_e5m2", "float16", "bfloat16", "float32", "float64")
INT_DTYPES = ("int4", "int8", "uint8", "int16", "int32", "int64")
ALL_DTYPES = FLOAT_DTYPES + INT_DTYPES

STORAGE = {
    "float8_e4m3": np.uint8, "float8_e5m2": np.uint8, "float16": np.float16, "bfloat16": np.uint16,
    "float32": np.float32, "float64": np.float64, "int4": np.int8, "int8": np.int8,
    "uint8": np.uint8, "int16": np.int16, "int32": np.int32, "int64": np.int64,
}


def f32_to_bf16_bits(x: np.ndarray) -> np.ndarray:
    """Round-to-nearest-even truncation of float32 to bfloat16 codes (non-NaN inputs)."""
    u = np.ascontiguousarray(x, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = (u + 0x7FFF + ((u >> 16) & 1)) >> 16
    return r.astype(np.uint16)


def bf16_bits_to_f32(b: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32)


def mixture(rng: np.random.Generator, shape) -> np.ndarray:
    n = int(np.prod(shape))
    pick = rng.random(n)
    v = np.where(pick < 0.5, rng.uniform(-10, 10, n),
                 np.where(pick < 0.75, rng.uniform(-1000, 1000, n), rng.uniform(-0.01, 0.01, n)))
    return v.reshape(shape)


def make(rng: np.random.Generator, shape, dtype: str, lo=None, hi=None) -> np.ndarray:
    """Random tensor of `dtype`; lo/hi switch to a plain uniform range."""
    if dtype in ("float8_e4m3", "float8_e5m2") and lo is None:
        return rng.integers(0, 256, size=shape, dtype=np.uint8)
    if dtype in INT_DTYPES:
        if lo is None:
            lo, hi = {"int4": (-7, 7), "int8": (-120, 120), "uint8": (0, 250)}.get(dtype, (-1000, 1000))
        return rng.integers(lo, hi + 1, size=shape).astype(STORAGE[dtype])
    v = mixture(rng, shape) if lo is None else rng.uniform(lo, hi, size=shape)
    return from_f64(v, dtype)


def from_f64(v: np.ndarray, dtype: str) -> np.ndarray:
    """Encode float64 values into the storage of `dtype` (IEEE rounding; test inputs only)."""
    v = np.asarray(v, dtype=np.float64)
    if dtype == "float64":
        return v.copy()
    if dtype == "float32":
        return v.astype(np.float32)
    if dtype == "float16":
        return v.astype(np.float32).astype(np.float16)
    if dtype == "bfloat16":
        return f32_to_bf16_bits(v.astype(np.float32))
    if dtype in ("float8_e4m3", "float8_e5m2"):
        import ml_dtypes
        t = ml_dtypes.float8_e4m3fn if dtype == "float8_e4m3" else ml_dtypes.float8_e5m2
        return v.astype(np.float32).astype(t).view(np.uint8)
    return np.rint(v).astype(STORAGE[dtype])


def to_f64(a: np.ndarray, dtype: str) -> np.ndarray:
    """Decode storage to float64 for error measurements."""
    if dtype == "bfloat16":
        return bf16_bits_to_f32(a).astype(np.float64)
    if dtype in ("float8_e4m3", "float8_e5m2"):
        import ml_dtypes
        t = ml_dtypes.float8_e4m3fn if dtype == "float8_e4m3" else ml_dtypes.float8_e5m2
        return np.ascontiguousarray(a, dtype=np.uint8).view(t).astype(np.float64)
    if dtype == "int4":
        lo = np.asarray(a, dtype=np.int8) & 0x0F
        return np.where(lo & 8, lo - 16, lo).astype(np.float64)
    return np.asarray(a).astype(np.float64)


def is_nan_code(a: np.ndarray, dtype: str) -> np.ndarray:
    if dtype in INT_DTYPES:
        return np.zeros(np.shape(a), dtype=bool)
    return np.isnan(to_f64(a, dtype))


def assert_same_codes(got: np.ndarray, want: np.ndarray, dtype: str, what: str = "") -> None:
    """Bit equality, except that any NaN matches any NaN (payload and sign of a NaN are
    platform detail; the reference's own checker accepts NaN<->NaN, numerical_correctness.py:190-255)."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    g = got.view(np.uint8) if got.dtype == np.bool_ else got
    same = g.view(_bits(g.dtype)) == want.view(_bits(want.dtype))
    if same.all():
        return
    both_nan = is_nan_code(got, dtype) & is_nan_code(want, dtype)
    bad = ~(same | both_nan)
    if bad.any():
        idx = np.argwhere(bad)[:5]
        detail = ", ".join(f"{tuple(i)}: got {got[tuple(i)]!r} want {want[tuple(i)]!r}" for i in idx)
        raise AssertionError(f"{what}: {int(bad.sum())} of {bad.size} codes differ ({detail})")


def _bits(dt):
    return {1: np.uint8, 2: np.uint16, 4: np.uint32, 8: np.uint64}[np.dtype(dt).itemsize]
