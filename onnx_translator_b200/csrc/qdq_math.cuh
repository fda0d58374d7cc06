// The arithmetic of QuantizeLinear (tensor_ops.c:999-1016), shared by the elementwise kernel and by
// the convolution that quantises its input on the fly.
#pragma once

#include "common.cuh"

namespace tops {

// ---- Quantize ------------------------------------------------------------------------------------------
// Reference arithmetic: r = (s != 0) ? rint(x / s) + z : z, all in double, then the generic store
// (integers: rint again + saturate; fp8: encode the integer-valued r).
//
// Fast path (x, s exact in float32; z a small integer): rint of the DOUBLE quotient equals rintf of
// the correctly rounded FLOAT quotient unless a half-integer lies within one float ulp of it; only
// those rare elements (and |q| >= 2^22) take the double division.
//
// The quotient itself is never needed, only its rounding, so the fast path does not divide at all:
// q ~ x * (1/s) with an approximate reciprocal is within 2^-21 |q| of x / s; adding and subtracting
// 1.5 * 2^23 rounds it to the nearest integer r (ties to even) and leaves r in the low mantissa
// bits.  r equals rint(x / s) -- for the exact quotient and for its double rounding alike --
// whenever q is further than 2^-19 |q| from a tie; the rest (about 1e-5 of the elements for
// |q| ~ 50, plus s == 0, non-finite x and |q| >= 2^21) take the double division.
// The approximate reciprocal the fast paths multiply by.  The hardware divide returns 0 for |s| above 2^126
// (a subnormal reciprocal), which would pass the tie test with a quotient of 0: a NaN sends those
// elements to the exact division instead.
__device__ __forceinline__ float quantize_reciprocal(float s) {
    return fabsf(s) < 8.5e37f ? __fdividef(1.0f, s) : __int_as_float(0x7FC00000);
}
// Returns rint(x / s) + z as an integer; `ok` tells whether the fast path was conclusive.
__device__ __forceinline__ int quantize_round_fast(float x, float inv_s, int z, bool& ok) {
    const float q = __fmul_rn(x, inv_s);
    const float t = __fadd_rn(q, 12582912.0f);
    const float r = __fsub_rn(t, 12582912.0f);
    const float aq = fabsf(q);
    ok = (aq < 2097152.0f) && (__fsub_rn(0.5f, fabsf(__fsub_rn(q, r))) > aq * 1.9073486e-6f);
    return (__float_as_int(t) - 0x4B400000) + z;
}
// 8-bit outputs with an 8-bit zero point: the same rounding and the same tie margin (2^-19 |q|,
// folded into one multiply-add, which also sends |q| >= 2^18 to the double division: the margin
// alone reaches 0.5 there).
// `z_minus_magic` = z - 0x4B400000, the same for every element of a run with one zero point.
__device__ __forceinline__ int quantize_round_8bit(float x, float inv_s, int z_minus_magic, bool& ok) {
    const float q = __fmul_rn(x, inv_s);
    const float t = __fadd_rn(q, 12582912.0f);
    const float d = __fsub_rn(q, __fsub_rn(t, 12582912.0f));
    ok = fmaf(fabsf(q), 1.9073486e-6f, fabsf(d)) < 0.5f;      // false too for |q| >= 2^18 (the margin alone is 0.5 there), Inf, NaN
    return __float_as_int(t) + z_minus_magic;
}
// The reference's arithmetic, element by element.
template <int DO>
__device__ __forceinline__ typename Storage<DO>::type quantize_exact(double x, double s, double z) {
    double r = z;
    if (s != 0.0) r = __dadd_rn(rint(__ddiv_rn(x, s)), z);
    return from_f64<DO>(r);
}


// The 8-bit code of one float32 value minus the zero point, i.e. the integer level the dequantised value is a multiple of,
// as a float (exact: |level| <= 255), without leaving the float pipe on the fast path: the rounded
// quotient is already a float integer, the saturation limits are float integers too.
template <int DO>
__device__ __forceinline__ float quantize_level_8bit(float x, float s, float inv_s, float zf) {
    const float q = __fmul_rn(x, inv_s);
    const float t = __fadd_rn(q, 12582912.0f);
    const float r = __fsub_rn(t, 12582912.0f);
    const float d = __fsub_rn(q, r);
    const bool ok = fmaf(fabsf(q), 1.9073486e-6f, fabsf(d)) < 0.5f;     // false too for |q| >= 2^18, Inf, NaN
    if (!ok) return (float)((int)quantize_exact<DO>((double)x, (double)s, (double)zf)) - zf;
    constexpr float lo = DO == DTYPE_INT8 ? -128.0f : 0.0f, hi = DO == DTYPE_INT8 ? 127.0f : 255.0f;
    return __fsub_rn(fminf(fmaxf(__fadd_rn(r, zf), lo), hi), zf);
}

// The same level by the reference's double division alone, kept OUT of line: the tensor-core epilogues call it only
// for the rare values their fast rounding cannot decide, and inlining sixteen double divisions into an epilogue that
// a handful of warps run would triple its code size for nothing.
static __device__ __noinline__ float quantize_level_exact(float x, float s, float zf, int is_signed) {
    const int code = is_signed ? (int)quantize_exact<DTYPE_INT8>((double)x, (double)s, (double)zf)
                               : (int)quantize_exact<DTYPE_UINT8>((double)x, (double)s, (double)zf);
    return (float)code - zf;
}

}  // namespace tops
