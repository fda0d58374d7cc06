// Broadcast Add / Sub / Mul / Div (tensor_ops.c:610-684 integer outputs, 864-997 dispatch).
// Each of the four operators is compiled in its own translation unit from this template.
//
// Arithmetic classes, chosen by the OUTPUT dtype exactly as the reference does:
//   integer output  -> both inputs to int64 (float inputs rounded to nearest-even first), the
//                      operator in wrapping int64, saturating store.  When both inputs are at
//                      most 16 bits wide the same result is formed in int32.
//   float64 output, or an input that float32 cannot hold exactly (int32, int64, float64)
//                   -> double arithmetic, one further rounding on store.
//   otherwise       -> float32 arithmetic with IEEE rounding: identical to "double, then round
//                      to float32" for + - * / because 53 >= 2*24 + 2.
#pragma once

#include "elementwise.cuh"

namespace tops {

enum BinaryOp { kAdd = 0, kSub = 1, kMul = 2, kDiv = 3, kMax = 4, kMin = 5, kPow = 6 };   // Max / Min / Pow: tensor_ops.c:1351-1403

template <int OP> __device__ __forceinline__ long long int_op64(long long a, long long b) {
    if constexpr (OP == kAdd) return (long long)((unsigned long long)a + (unsigned long long)b);
    else if constexpr (OP == kSub) return (long long)((unsigned long long)a - (unsigned long long)b);
    else if constexpr (OP == kMul) return (long long)((unsigned long long)a * (unsigned long long)b);
    else if constexpr (OP == kMax) return a > b ? a : b;
    else if constexpr (OP == kMin) return a < b ? a : b;
    else {
        if (b == 0) return a >= 0 ? 0x7FFFFFFFFFFFFFFFll : (long long)0x8000000000000000ull;
        if (b == -1) return (long long)(0ull - (unsigned long long)a);          // avoids INT64_MIN / -1
        // both operands fit 32 bits in nearly every real tensor: use the cheap divider then
        if (a == (int)a && b == (int)b) return (long long)((int)a / (int)b);
        return a / b;
    }
}
// Truncated quotient of two integers below 2^16 in magnitude (given as floats) without the integer
// divider: a * (1/b) is within 2^-22 relative of the quotient; scaling by 1 + 2^-20 lifts an exact
// quotient to at least itself, and never reaches the next integer, because a quotient that is not
// an integer is at least |q| * 2^-16 away from one.  Truncation then gives a / b.  Division by
// zero yields the extreme of the sign of a, as the reference does.
__device__ __forceinline__ int narrow_int_quotient(float a, float b) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(b));
    const int q = __float2int_rz(__fmul_rn(__fmul_rn(a, r), 1.00000095367431640625f));
    return b == 0.0f ? (a >= 0.0f ? 0x7FFFFFFF : (int)0x80000000) : q;
}
template <int OP> __device__ __forceinline__ int int_op32(int a, int b) {      // inputs within 16 bits
    if constexpr (OP == kAdd) return a + b;
    else if constexpr (OP == kSub) return a - b;
    else if constexpr (OP == kMul) return a * b;
    else if constexpr (OP == kMax) return a > b ? a : b;
    else if constexpr (OP == kMin) return a < b ? a : b;
    else return narrow_int_quotient((float)a, (float)b);
}
template <int OP> __device__ __forceinline__ float float_op32(float a, float b) {
    if constexpr (OP == kAdd) return __fadd_rn(a, b);
    else if constexpr (OP == kSub) return __fsub_rn(a, b);
    else if constexpr (OP == kMul) return __fmul_rn(a, b);
    else if constexpr (OP == kMax) return a > b ? a : b;       // a NaN on either side yields b, as the reference's ternary
    else if constexpr (OP == kMin) return a < b ? a : b;
    else return __fdiv_rn(a, b);
}
template <int OP> __device__ __forceinline__ double float_op64(double a, double b) {
    if constexpr (OP == kAdd) return __dadd_rn(a, b);
    else if constexpr (OP == kSub) return __dsub_rn(a, b);
    else if constexpr (OP == kMul) return __dmul_rn(a, b);
    else if constexpr (OP == kMax) return a > b ? a : b;
    else if constexpr (OP == kMin) return a < b ? a : b;
    else if constexpr (OP == kPow) return pow(a, b);
    else return __ddiv_rn(a, b);
}

template <int DA, int DB, int DO, int OP>
__device__ __forceinline__ typename Storage<DO>::type
binary_elem(typename Storage<DA>::type sa, typename Storage<DB>::type sb) {
    if constexpr (OP == kPow) {                                  // always double, then the generic store
        return from_f64<DO>(pow(to_f64<DA>(sa), to_f64<DB>(sb)));
    } else if constexpr (dtype_is_int(DO)) {
        if constexpr (dtype_is_narrow_int(DA) && dtype_is_narrow_int(DB) && DO != DTYPE_INT64) {
            return from_i32<DO>(int_op32<OP>(to_i32_narrow<DA>(sa), to_i32_narrow<DB>(sb)));
        } else {
            return from_i64<DO>(int_op64<OP>(to_i64<DA>(sa), to_i64<DB>(sb)));
        }
    } else if constexpr (DO == DTYPE_FLOAT64 || !dtype_exact_in_f32(DA) || !dtype_exact_in_f32(DB)) {
        return from_f64<DO>(float_op64<OP>(to_f64<DA>(sa), to_f64<DB>(sb)));
    } else {
        return from_f32<DO>(float_op32<OP>(to_f32<DA>(sa), to_f32<DB>(sb)));
    }
}

template <int DA, int DB, int DO, int OP, bool ALIGNED>
struct BinaryBody {
    static constexpr int kV = vec_width(dtype_bytes(DA), dtype_bytes(DB), dtype_bytes(DO));
    static constexpr bool kMixedWidths = dtype_bytes(DA) != dtype_bytes(DB) || dtype_bytes(DB) != dtype_bytes(DO);
    static constexpr bool kWideDivide = OP == kDiv && (DO == DTYPE_FLOAT64 || (DO == DTYPE_FLOAT32 && DA == DTYPE_FLOAT32 && DB == DTYPE_FLOAT32));
    static constexpr int kGroups = kWideDivide ? 4 : kMixedWidths ? 2 : 0;     // 0: run kernel
    struct Regs {
        Run<typename Storage<DA>::type, kV> ra;
        Run<typename Storage<DB>::type, kV> rb;
    };
    Geo3 g;
    Op3 a, b;
    void* out;
    __device__ __forceinline__ void load(uint32_t i0, uint32_t nv, Regs& r) const {
        const Coord3 c = g.simple ? Coord3{0, 0, 0} : coords_of(g, i0);
        fetch3<DA, kV, ALIGNED>(g, a, i0, nv, c, r.ra);
        fetch3<DB, kV, ALIGNED>(g, b, i0, nv, c, r.rb);
    }
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        Regs r;
        load(i0, nv, r);
        finish(i0, nv, r);
    }
    __device__ __forceinline__ void finish(uint32_t i0, uint32_t nv, const Regs& r) const {
        const Run<typename Storage<DA>::type, kV>& ra = r.ra;
        const Run<typename Storage<DB>::type, kV>& rb = r.rb;
        Run<typename Storage<DO>::type, kV> ro;
        constexpr bool int_lane = OP != kPow && dtype_is_int(DO) && DO != DTYPE_INT64 && dtype_is_narrow_int(DA) && dtype_is_narrow_int(DB) &&
                                  dtype_is_narrow_int(DO);
        constexpr bool float_lane = OP != kPow && !dtype_is_int(DO) && DO != DTYPE_FLOAT64 && dtype_exact_in_f32(DA) && dtype_exact_in_f32(DB);
        if constexpr (int_lane) {
            int v[kV];
            if constexpr (OP == kDiv && kV % 4 == 0 && (DA == DTYPE_INT8 || DA == DTYPE_UINT8) && (DB == DTYPE_INT8 || DB == DTYPE_UINT8)) {
                float fa[kV], fb[kV];                     // bytes to float on the integer pipe, no conversion unit
                decode_floats<DA, kV>(ra, fa);
                decode_floats<DB, kV>(rb, fb);
                #pragma unroll
                for (int j = 0; j < kV; j++) v[j] = narrow_int_quotient(fa[j], fb[j]);
            } else {
                #pragma unroll
                for (int j = 0; j < kV; j++) v[j] = int_op32<OP>(to_i32_narrow<DA>(ra.v[j]), to_i32_narrow<DB>(rb.v[j]));
            }
            encode_ints<DO, kV>(v, ro);
        } else if constexpr (float_lane) {
            float fa[kV], fb[kV];
            decode_floats<DA, kV>(ra, fa);
            decode_floats<DB, kV>(rb, fb);
            #pragma unroll
            for (int j = 0; j < kV; j++) fa[j] = float_op32<OP>(fa[j], fb[j]);
            encode_floats<DO, kV>(fa, ro);
        } else {
            #pragma unroll
            for (int j = 0; j < kV; j++) ro.v[j] = binary_elem<DA, DB, DO, OP>(ra.v[j], rb.v[j]);
        }
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
};

// Any dtype triple and any rank: one element per run, dtypes switched at run time.
template <int OP>
struct BinaryGenericBody {
    static constexpr int kV = 1;
    static constexpr int kGroups = 0;
    Geometry g;
    Operand a, b;
    void* out;
    int da, db, dout;
    __device__ __forceinline__ void operator()(uint32_t i, uint32_t) const {
        uint32_t p;
        const uint32_t ia = a.flat ? i : operand_offset(g, a, i, p);
        const uint32_t ib = b.flat ? i : operand_offset(g, b, i, p);
        if (OP != kPow && dtype_is_int(dout)) {
            store_i64_rt(out, dout, i, int_op64<OP>(load_i64_rt(a.ptr, da, ia), load_i64_rt(b.ptr, db, ib)));
        } else {
            store_f64_rt(out, dout, i, float_op64<OP>(load_f64_rt(a.ptr, da, ia), load_f64_rt(b.ptr, db, ib)));
        }
    }
};

template <int OP>
static bool binary_generic_slab(const char* name, const Slab& s, int da, int db, int dout) {
    BinaryGenericBody<OP> body{s.geom, s.ops[0], s.ops[1], s.out, da, db, dout};
    return launch_body(name, body, s.n);
}

template <int DA, int DB, int DO, int OP>
static bool binary_typed(const char* name, const Geometry& geom, Operand* ops, Tensor* o) {
    const int bytes[2] = {dtype_bytes(DA), dtype_bytes(DB)};
    return for_each_slab(name, geom, ops, bytes, 2, o->data, dtype_bytes(DO), o->size, [&](const Slab& s) {
        if (!s.fits3) return binary_generic_slab<OP>(name, s, DA, DB, DO);
        constexpr int V = BinaryBody<DA, DB, DO, OP, true>::kV;
        if (slab_aligned(s, 2, bytes, dtype_bytes(DO), V)) {
            BinaryBody<DA, DB, DO, OP, true> body{s.geo3, s.ops3[0], s.ops3[1], s.out};
            return launch_body(name, body, s.n);
        }
        BinaryBody<DA, DB, DO, OP, false> body{s.geo3, s.ops3[0], s.ops3[1], s.out};
        return launch_body(name, body, s.n);
    });
}

template <int OP>
static void binary_forward(const char* name, const Tensor* a, const Tensor* b, Tensor* o) {
    if (!a || !b || !o || !a->data || !b->data || !o->data) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor", name);
        zero_fill(o);
        return;
    }
    const int da = (int)a->dtype, db = (int)b->dtype, dout = (int)o->dtype;
    if (!dtype_valid(da) || !dtype_valid(db) || !dtype_valid(dout)) { set_error(TOPS_ERR_INVALID, "%s: bad dtype", name); return; }
    Geometry geom;
    Operand ops[2];
    const ShapeView out{o->shape, o->ndim, o->size};
    const ShapeView ins[2] = {{a->shape, a->ndim, a->size}, {b->shape, b->ndim, b->size}};
    if (!plan_broadcast(out, ins, 2, &geom, ops)) {
        set_error(TOPS_ERR_INVALID, "%s: operand shapes do not broadcast to the output shape", name);
        zero_fill(o);
        return;
    }
    ops[0].ptr = a->data;
    ops[1].ptr = b->data;

    bool done = false;
#define TOPS_COMBO(A, B, O) if (!done && da == A && db == B && dout == O) { binary_typed<A, B, O, OP>(name, geom, ops, o); done = true; }
#define TOPS_SAME(T) TOPS_COMBO(T, T, T)
    TOPS_SAME(DTYPE_FLOAT32) TOPS_SAME(DTYPE_FLOAT16) TOPS_SAME(DTYPE_BFLOAT16) TOPS_SAME(DTYPE_FLOAT64)
    TOPS_SAME(DTYPE_INT32) TOPS_SAME(DTYPE_INT8) TOPS_SAME(DTYPE_UINT8) TOPS_SAME(DTYPE_INT16)
    TOPS_SAME(DTYPE_INT64) TOPS_SAME(DTYPE_INT4) TOPS_SAME(DTYPE_FLOAT8_E4M3) TOPS_SAME(DTYPE_FLOAT8_E5M2)
    TOPS_COMBO(DTYPE_INT8, DTYPE_FLOAT32, DTYPE_FLOAT32) TOPS_COMBO(DTYPE_FLOAT32, DTYPE_INT8, DTYPE_FLOAT32)
    TOPS_COMBO(DTYPE_INT32, DTYPE_FLOAT16, DTYPE_FLOAT64) TOPS_COMBO(DTYPE_FLOAT16, DTYPE_INT32, DTYPE_FLOAT64)
    TOPS_COMBO(DTYPE_BFLOAT16, DTYPE_FLOAT32, DTYPE_FLOAT32) TOPS_COMBO(DTYPE_FLOAT32, DTYPE_BFLOAT16, DTYPE_FLOAT32)
    TOPS_COMBO(DTYPE_FLOAT16, DTYPE_FLOAT32, DTYPE_FLOAT32) TOPS_COMBO(DTYPE_FLOAT32, DTYPE_FLOAT16, DTYPE_FLOAT32)
#undef TOPS_SAME
#undef TOPS_COMBO
    if (!done) {
        const int bytes[2] = {dtype_bytes(da), dtype_bytes(db)};
        for_each_slab(name, geom, ops, bytes, 2, o->data, dtype_bytes(dout), o->size,
                      [&](const Slab& s) { return binary_generic_slab<OP>(name, s, da, db, dout); });
    }
    finish_op();
}

}  // namespace tops
