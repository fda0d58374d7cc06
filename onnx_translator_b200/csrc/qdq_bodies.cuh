// The typed bodies of QuantizeLinear / DequantizeLinear (tensor_ops.c:999-1034) for the elementwise engine.
// Each computes one run from registers to registers (`compute`) and stores it (`finish`), so that a fused body
// can chain them without a trip through memory.
#pragma once

#include "elementwise.cuh"
#include "qdq_math.cuh"

namespace tops {

// ---- Quantize (arithmetic: qdq_math.cuh) -------------------------------------------------------------
template <int DX, int DS, int DZ, int DO, bool ALIGNED>
struct QuantizeBody {
    static constexpr int kV = vec_width(dtype_bytes(DX), dtype_bytes(DO), dtype_bytes(DO), 64);
    using Codes = Run<typename Storage<DO>::type, kV>;
    static constexpr int kGroups = 0;
    struct Regs {
        Run<typename Storage<DX>::type, kV> rx;
        Run<typename Storage<DS>::type, kV> rs;
        Run<typename Storage<DZ>::type, kV> rz;
    };
    Geo3 g;
    Op3 x, s, z;
    void* out;
    __device__ __forceinline__ void load(uint32_t i0, uint32_t nv, Regs& r) const {
        const Coord3 c = g.simple ? Coord3{0, 0, 0} : coords_of(g, i0);
        fetch3<DX, kV, ALIGNED>(g, x, i0, nv, c, r.rx);
        fetch3<DS, kV, ALIGNED>(g, s, i0, nv, c, r.rs);
        fetch3<DZ, kV, ALIGNED>(g, z, i0, nv, c, r.rz);
    }
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        Regs r;
        load(i0, nv, r);
        finish(i0, nv, r);
    }
    __device__ __forceinline__ void finish(uint32_t i0, uint32_t nv, const Regs& r) const {
        Codes ro;
        compute(r, ro);
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
    // The codes of one run, left in registers (the fused round trip dequantises them straight away).
    __device__ __forceinline__ void compute(const Regs& r, Codes& ro) const {
        const Run<typename Storage<DX>::type, kV>& rx = r.rx;
        const Run<typename Storage<DS>::type, kV>& rs = r.rs;
        const Run<typename Storage<DZ>::type, kV>& rz = r.rz;
        if constexpr (dtype_exact_in_f32(DX) && dtype_exact_in_f32(DS) && dtype_is_narrow_int(DZ)) {
            float fx[kV];
            decode_floats<DX, kV>(rx, fx);
            int v[kV];
            bool all_ok = true;
            const bool uniform_scale = ALIGNED && !g.simple && s.st2 == 0;    // one scale for the whole run
            float inv = uniform_scale ? quantize_reciprocal(to_f32<DS>(rs.v[0])) : 0.0f;
            constexpr bool kEightBit = (DO == DTYPE_INT8 || DO == DTYPE_UINT8 || DO == DTYPE_FLOAT8_E4M3 || DO == DTYPE_FLOAT8_E5M2) &&
                                       (DZ == DTYPE_INT8 || DZ == DTYPE_UINT8);
            constexpr bool kFp8Out = DO == DTYPE_FLOAT8_E4M3 || DO == DTYPE_FLOAT8_E5M2;
            if constexpr (kEightBit && kFp8Out && kV % 2 == 0) {
                // fp8 targets: the rounded quotient plus the zero point stays a float (an exact integer)
                // and is encoded two at a time by the hardware convert, which agrees with the reference's
                // encoder for integer values below its overflow threshold (e5m2: 61440 -> Inf) -- larger
                // quotients take the element-wise path below.
                float fr[kV];
                constexpr float kLimit = DO == DTYPE_FLOAT8_E5M2 ? 57000.0f : 262144.0f;    // e4m3: implied by the tie test
                const bool uniform_zero = ALIGNED && !g.simple && z.st2 == 0;     // one int -> float conversion per run then
                const float zf0 = (float)to_i32_narrow<DZ>(rz.v[0]);
                #pragma unroll
                for (int j = 0; j < kV; j++) {
                    if (!uniform_scale) inv = quantize_reciprocal(to_f32<DS>(rs.v[j]));
                    const float q = __fmul_rn(fx[j], inv);
                    const float t = __fadd_rn(q, 12582912.0f);
                    const float rq = __fsub_rn(t, 12582912.0f);
                    const float d = __fsub_rn(q, rq);
                    all_ok = all_ok & (fmaf(fabsf(q), 1.9073486e-6f, fabsf(d)) < 0.5f);
                    if constexpr (DO == DTYPE_FLOAT8_E5M2) all_ok = all_ok & (fabsf(q) < kLimit);
                    fr[j] = __fadd_rn(rq, uniform_zero ? zf0 : (float)to_i32_narrow<DZ>(rz.v[j]));
                }
                if (all_ok) {
                    #pragma unroll
                    for (int j = 0; j < kV; j += 2) {
                        const __nv_fp8x2_storage_t two = __nv_cvt_float2_to_fp8x2(make_float2(fr[j], fr[j + 1]), __NV_SATFINITE,
                                                                                  DO == DTYPE_FLOAT8_E4M3 ? __NV_E4M3 : __NV_E5M2);
                        *reinterpret_cast<uint16_t*>(&ro.v[j]) = (uint16_t)two;
                    }
                    return;
                }
                #pragma unroll
                for (int j = 0; j < kV; j++) v[j] = 0;
                all_ok = false;
            } else if (kEightBit && uniform_scale && z.st2 == 0) {
                const int zm = to_i32_narrow<DZ>(rz.v[0]) - 0x4B400000;
                #pragma unroll
                for (int j = 0; j < kV; j++) {
                    bool ok;
                    v[j] = quantize_round_8bit(fx[j], inv, zm, ok);
                    all_ok = all_ok & ok;
                }
            } else if (kEightBit) {
                #pragma unroll
                for (int j = 0; j < kV; j++) {
                    if (!uniform_scale) inv = quantize_reciprocal(to_f32<DS>(rs.v[j]));
                    bool ok;
                    v[j] = quantize_round_8bit(fx[j], inv, to_i32_narrow<DZ>(rz.v[j]) - 0x4B400000, ok);
                    all_ok = all_ok & ok;
                }
            } else {
                #pragma unroll
                for (int j = 0; j < kV; j++) {
                    if (!uniform_scale) inv = quantize_reciprocal(to_f32<DS>(rs.v[j]));
                    bool ok;
                    v[j] = quantize_round_fast(fx[j], inv, to_i32_narrow<DZ>(rz.v[j]), ok);
                    all_ok = all_ok && ok;
                }
            }
            if (all_ok) {
                if constexpr (DO == DTYPE_INT8 || DO == DTYPE_UINT8) {
                    encode_ints<DO, kV>(v, ro);
                } else {
                    float fr[kV];
                    #pragma unroll
                    for (int j = 0; j < kV; j++) fr[j] = (float)v[j];       // |v| < 2^22: exact
                    encode_floats<DO, kV>(fr, ro);
                }
            } else {
                #pragma unroll
                for (int j = 0; j < kV; j++)
                    ro.v[j] = quantize_exact<DO>((double)fx[j], to_f64<DS>(rs.v[j]), to_f64<DZ>(rz.v[j]));
            }
        } else {
            #pragma unroll
            for (int j = 0; j < kV; j++)
                ro.v[j] = quantize_exact<DO>(to_f64<DX>(rx.v[j]), to_f64<DS>(rs.v[j]), to_f64<DZ>(rz.v[j]));
        }
    }
};

// ---- Dequantize ----------------------------------------------------------------------------------------
// Reference arithmetic: (x - z) * s in double, rounded once on store.  In float32 the same bits
// come out whenever x - z is exact in float32 (8-bit integers, e4m3 codes, any x with z == 0):
// the double product of a <= 24-bit difference and a 24-bit scale is exact, so a single
// correctly rounded float multiply reproduces "exact product, one rounding".
template <int DX, int DS, int DZ, int DO, bool ALIGNED, int RUN>
struct DequantizeBodyN {
    static constexpr bool kDiffExact = dtype_exact_in_f32(DX) && dtype_exact_in_f32(DZ) && dtype_exact_in_f32(DS) &&
        DX != DTYPE_FLOAT8_E5M2 && DZ != DTYPE_FLOAT8_E5M2 && DX != DTYPE_FLOAT16 && DZ != DTYPE_FLOAT16 &&
        DX != DTYPE_BFLOAT16 && DZ != DTYPE_BFLOAT16 && DX != DTYPE_FLOAT32 && DZ != DTYPE_FLOAT32 &&
        DO != DTYPE_FLOAT64 && !dtype_is_int(DO);
    static constexpr int kV = RUN ? RUN : vec_width(dtype_bytes(DX), dtype_bytes(DO), dtype_bytes(DO));     // RUN: run length imposed by a fused body
    static constexpr int kGroups = 2;
    using Values = Run<typename Storage<DO>::type, kV>;
    struct Regs {
        Run<typename Storage<DX>::type, kV> rx;
        Run<typename Storage<DS>::type, kV> rs;
        Run<typename Storage<DZ>::type, kV> rz;
    };
    Geo3 g;
    Op3 x, s, z;
    void* out;
    __device__ __forceinline__ void load(uint32_t i0, uint32_t nv, Regs& r) const {
        const Coord3 c = g.simple ? Coord3{0, 0, 0} : coords_of(g, i0);
        fetch3<DX, kV, ALIGNED>(g, x, i0, nv, c, r.rx);
        fetch3<DS, kV, ALIGNED>(g, s, i0, nv, c, r.rs);
        fetch3<DZ, kV, ALIGNED>(g, z, i0, nv, c, r.rz);
    }
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        Regs r;
        load(i0, nv, r);
        finish(i0, nv, r);
    }
    __device__ __forceinline__ void finish(uint32_t i0, uint32_t nv, const Regs& r) const {
        Values ro;
        compute(r.rx, r.rs, r.rz, nv == (uint32_t)kV, ro);
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
    // `full`: the run is complete (its scale and zero point registers hold the run's own values throughout).
    __device__ __forceinline__ void compute(const Run<typename Storage<DX>::type, kV>& rx, const Run<typename Storage<DS>::type, kV>& rs,
                                            const Run<typename Storage<DZ>::type, kV>& rz, bool full, Values& ro) const {
        if constexpr (kDiffExact && (DX == DTYPE_INT8 || DX == DTYPE_UINT8) && kV % 4 == 0) {
            // one scale and one zero point for the whole run: the byte is placed in the low mantissa
            // byte of 2^23 and (2^23 + offset + z) is subtracted in one exact step
            if (ALIGNED && full && !g.simple && s.st2 == 0 && z.st2 == 0) {
                const float fs = to_f32<DS>(rs.v[0]);
                const float base = __fadd_rn(DX == DTYPE_INT8 ? 8388736.0f : 8388608.0f, to_f32<DZ>(rz.v[0]));
                float f[kV];
                #pragma unroll
                for (int j = 0; j < kV; j += 4) {
                    uint32_t w = *reinterpret_cast<const uint32_t*>(&rx.v[j]);
                    if (DX == DTYPE_INT8) w ^= 0x80808080u;
                    f[j]     = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), base), fs);
                    f[j + 1] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)), base), fs);
                    f[j + 2] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)), base), fs);
                    f[j + 3] = __fmul_rn(__fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)), base), fs);
                }
                encode_floats<DO, kV>(f, ro);
                return;
            }
        }
        if constexpr (kDiffExact) {
            float fx[kV], fz[kV], f[kV];
            decode_floats<DX, kV>(rx, fx);
            decode_floats<DZ, kV>(rz, fz);
            #pragma unroll
            for (int j = 0; j < kV; j++) f[j] = __fmul_rn(__fsub_rn(fx[j], fz[j]), to_f32<DS>(rs.v[j]));
            encode_floats<DO, kV>(f, ro);
            return;
        }
        if constexpr (!kDiffExact && dtype_exact_in_f32(DX) && dtype_exact_in_f32(DS) && dtype_exact_in_f32(DZ) &&
                      DO != DTYPE_FLOAT64 && !dtype_is_int(DO)) {
            // e.g. e5m2 or float16 codes: with a zero point of zero the product is a single rounding too
            bool zero_points_zero = true;
            #pragma unroll
            for (int j = 0; j < kV; j++) zero_points_zero = zero_points_zero && to_f32<DZ>(rz.v[j]) == 0.0f;
            if (zero_points_zero) {
                float fx[kV], f[kV];
                decode_floats<DX, kV>(rx, fx);
                #pragma unroll
                for (int j = 0; j < kV; j++) f[j] = __fmul_rn(fx[j], to_f32<DS>(rs.v[j]));
                encode_floats<DO, kV>(f, ro);
                return;
            }
        }
        #pragma unroll
        for (int j = 0; j < kV; j++) {
            if constexpr (kDiffExact) {
                ro.v[j] = typename Storage<DO>::type(0);        // handled above
            } else if constexpr (dtype_exact_in_f32(DX) && dtype_exact_in_f32(DS) && dtype_exact_in_f32(DZ) &&
                                 DO != DTYPE_FLOAT64 && !dtype_is_int(DO)) {
                const float zv = to_f32<DZ>(rz.v[j]);
                if (zv == 0.0f) {
                    ro.v[j] = from_f32<DO>(__fmul_rn(to_f32<DX>(rx.v[j]), to_f32<DS>(rs.v[j])));
                } else {
                    const double d = __dsub_rn(to_f64<DX>(rx.v[j]), (double)zv);
                    ro.v[j] = from_f64<DO>(__dmul_rn(d, to_f64<DS>(rs.v[j])));
                }
            } else {
                const double d = __dsub_rn(to_f64<DX>(rx.v[j]), to_f64<DZ>(rz.v[j]));
                ro.v[j] = from_f64<DO>(__dmul_rn(d, to_f64<DS>(rs.v[j])));
            }
        }
    }
};

template <int DX, int DS, int DZ, int DO, bool ALIGNED> using DequantizeBody = DequantizeBodyN<DX, DS, DZ, DO, ALIGNED, 0>;

}  // namespace tops
