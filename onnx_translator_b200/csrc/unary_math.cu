// The one-line unary operators of the reference (tensor_ops.c:595-604 is their shared shape: read the
// element as a double, evaluate one libm expression, store like any operator result):
//   exp log sqrt sigmoid tanh (:1273-1286), neg reciprocal ceil floor (:1484-1493), sin tan atan (:1758-1760),
//   softplus softsign hard_swish acos asin cosh sinh asinh acosh atanh (:2622-2665), round erf (:3032-3035),
//   gelu (:3340).
// The expressions are evaluated in double here too, operation by operation (no fused multiply-add).
// neg, reciprocal, ceil, floor, sqrt, round, softsign and hard_swish consist of exactly rounded operations
// and are bit-identical (six of them are evaluated in float32 where that provably gives the same float32);
// the others call the CUDA double-precision functions, which like glibc's are
// accurate to about one unit in the last place of a DOUBLE, so float32 and narrower results agree except
// where the exact value lies within that distance of a rounding boundary.
#include "elementwise.cuh"

namespace tops {

enum MathOp { kExp, kLog, kSqrt, kSigmoid, kTanh, kNeg, kReciprocal, kCeil, kFloor, kSin, kTan, kAtan, kSoftplus, kSoftsign,
              kHardSwish, kAcos, kAsin, kCosh, kSinh, kAsinh, kAcosh, kAtanh, kRound, kErf, kGelu };

template <int OP> __device__ __forceinline__ double math_value(double v) {
    if constexpr (OP == kExp) return exp(v);
    else if constexpr (OP == kLog) return log(v);
    else if constexpr (OP == kSqrt) return sqrt(v);
    else if constexpr (OP == kSigmoid) return __ddiv_rn(1.0, __dadd_rn(1.0, exp(-v)));
    else if constexpr (OP == kTanh) return tanh(v);
    else if constexpr (OP == kNeg) return -v;
    else if constexpr (OP == kReciprocal) return __ddiv_rn(1.0, v);
    else if constexpr (OP == kCeil) return ceil(v);
    else if constexpr (OP == kFloor) return floor(v);
    else if constexpr (OP == kSin) return sin(v);
    else if constexpr (OP == kTan) return tan(v);
    else if constexpr (OP == kAtan) return atan(v);
    else if constexpr (OP == kSoftplus) return log(__dadd_rn(1.0, exp(v)));
    else if constexpr (OP == kSoftsign) return __ddiv_rn(v, __dadd_rn(1.0, fabs(v)));
    else if constexpr (OP == kHardSwish) return __dmul_rn(v, fmax(0.0, fmin(1.0, __dadd_rn(__ddiv_rn(v, 6.0), 0.5))));
    else if constexpr (OP == kAcos) return acos(v);
    else if constexpr (OP == kAsin) return asin(v);
    else if constexpr (OP == kCosh) return cosh(v);
    else if constexpr (OP == kSinh) return sinh(v);
    else if constexpr (OP == kAsinh) return asinh(v);
    else if constexpr (OP == kAcosh) return acosh(v);
    else if constexpr (OP == kAtanh) return atanh(v);
    else if constexpr (OP == kRound) return rint(v);
    else if constexpr (OP == kErf) return erf(v);
    else return __dmul_rn(__dmul_rn(0.5, v), __dadd_rn(1.0, erf(__dmul_rn(v, 0.70710678118654752440))));     // gelu
}

// Operators whose double expression, rounded to float32, equals the same operation done in float32:
// negation and the three roundings are exact, and for square root and division a result rounded to
// 53 bits and then to 24 equals the result rounded to 24 bits directly (53 >= 2 * 24 + 2).
template <int OP> __host__ __device__ constexpr bool math_exact_in_f32() {
    return OP == kNeg || OP == kCeil || OP == kFloor || OP == kRound || OP == kSqrt || OP == kReciprocal;
}
template <int OP> __device__ __forceinline__ float math_value_f32(float v) {
    if constexpr (OP == kNeg) return -v;
    else if constexpr (OP == kCeil) return ceilf(v);
    else if constexpr (OP == kFloor) return floorf(v);
    else if constexpr (OP == kRound) return rintf(v);
    else if constexpr (OP == kSqrt) return __fsqrt_rn(v);
    else if constexpr (OP == kReciprocal) return __fdiv_rn(1.0f, v);
    else return __double2float_rn(math_value<OP>((double)v));
}

// float32 / float16 / bfloat16 in and out: vector loads and stores, the value rounded to float32 first and
// then encoded, which is what the store of these types does with a double.
template <int OP, int DX, int DO, bool ALIGNED>
struct MathTypedBody {
    static constexpr int kV = vec_width(dtype_bytes(DX), dtype_bytes(DO), dtype_bytes(DO));
    static constexpr int kGroups = 0;
    struct Regs { Run<typename Storage<DX>::type, kV> in; };
    Geo3 g;
    Op3 x;
    void* out;
    __device__ __forceinline__ void load(uint32_t i0, uint32_t nv, Regs& r) const {
        fetch3<DX, kV, ALIGNED>(g, x, i0, nv, Coord3{0, 0, 0}, r.in);
    }
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        Regs r;
        load(i0, nv, r);
        finish(i0, nv, r);
    }
    __device__ __forceinline__ void finish(uint32_t i0, uint32_t nv, const Regs& r) const {
        float f[kV];
        decode_floats<DX, kV>(r.in, f);
        #pragma unroll
        for (int j = 0; j < kV; j++) f[j] = math_value_f32<OP>(f[j]);
        Run<typename Storage<DO>::type, kV> res;
        encode_floats<DO, kV>(f, res);
        put3<DO, kV, ALIGNED>(out, i0, nv, res);
    }
};

// Any dtype pair; the dtypes are uniform across the grid, so the switches inside load / store do not diverge.
template <int OP>
struct MathBody {
    static constexpr int kV = 1;
    static constexpr int kGroups = 0;
    const void* x;
    void* out;
    int dx, dout;
    __device__ __forceinline__ void operator()(uint32_t i, uint32_t) const {
        store_f64_rt(out, dout, i, math_value<OP>(load_f64_rt(x, dx, i)));
    }
};

template <int OP, int DT>
static bool math_typed(const char* name, const Tensor* x, Tensor* y) {
    Geometry geom;
    Operand op;
    const ShapeView out{y->shape, y->ndim, y->size}, in{x->shape, x->ndim, x->size};
    if (!plan_broadcast(out, &in, 1, &geom, &op)) return false;
    op.ptr = x->data;
    const int bytes[1] = {dtype_bytes(DT)};
    return for_each_slab(name, geom, &op, bytes, 1, y->data, dtype_bytes(DT), y->size, [&](const Slab& s) {
        constexpr int V = MathTypedBody<OP, DT, DT, true>::kV;
        if (slab_aligned(s, 1, bytes, dtype_bytes(DT), V)) {
            MathTypedBody<OP, DT, DT, true> b{s.geo3, s.ops3[0], s.out};
            return launch_body(name, b, s.n);
        }
        MathTypedBody<OP, DT, DT, false> b{s.geo3, s.ops3[0], s.out};
        return launch_body(name, b, s.n);
    });
}

template <int OP>
static void math_forward(const char* name, const Tensor* x, Tensor* y) {
    if (!x || !y || !x->data || !y->data || x->size != y->size) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor or size mismatch", name);
        zero_fill(y);
        return;
    }
    if (!dtype_valid((int)x->dtype) || !dtype_valid((int)y->dtype)) { set_error(TOPS_ERR_INVALID, "%s: bad dtype", name); return; }
    const int dx = (int)x->dtype, dout = (int)y->dtype;
    bool done = false;
    if (dx == dout && x->shape && y->shape) {
        if (dx == DTYPE_FLOAT32) done = math_typed<OP, DTYPE_FLOAT32>(name, x, y);
        else if (dx == DTYPE_FLOAT16) done = math_typed<OP, DTYPE_FLOAT16>(name, x, y);
        else if (dx == DTYPE_BFLOAT16) done = math_typed<OP, DTYPE_BFLOAT16>(name, x, y);
    }
    if (!done) {
        const size_t ex = (size_t)dtype_bytes(dx), eo = (size_t)dtype_bytes(dout);
        const size_t kSlab = 0x7FFFFF00ull;                        // 32-bit indices inside a launch
        for (size_t first = 0; first < x->size; first += kSlab) {
            const size_t n = x->size - first < kSlab ? x->size - first : kSlab;
            MathBody<OP> body{(const char*)x->data + first * ex, (char*)y->data + first * eo, dx, dout};
            if (!launch_body(name, body, n)) return;
        }
    }
    finish_op();
}

}  // namespace tops

using namespace tops;

#define TOPS_MATH_ENTRY(NAME, OP) TOPS_API void NAME(const Tensor* input, Tensor* output) { math_forward<OP>(#NAME, input, output); }
TOPS_MATH_ENTRY(exp_forward, kExp)
TOPS_MATH_ENTRY(log_forward, kLog)
TOPS_MATH_ENTRY(sqrt_forward, kSqrt)
TOPS_MATH_ENTRY(sigmoid_forward, kSigmoid)
TOPS_MATH_ENTRY(tanh_forward, kTanh)
TOPS_MATH_ENTRY(neg_forward, kNeg)
TOPS_MATH_ENTRY(reciprocal_forward, kReciprocal)
TOPS_MATH_ENTRY(ceil_forward, kCeil)
TOPS_MATH_ENTRY(floor_forward, kFloor)
TOPS_MATH_ENTRY(sin_forward, kSin)
TOPS_MATH_ENTRY(tan_forward, kTan)
TOPS_MATH_ENTRY(atan_forward, kAtan)
TOPS_MATH_ENTRY(softplus_forward, kSoftplus)
TOPS_MATH_ENTRY(softsign_forward, kSoftsign)
TOPS_MATH_ENTRY(hard_swish_forward, kHardSwish)
TOPS_MATH_ENTRY(acos_forward, kAcos)
TOPS_MATH_ENTRY(asin_forward, kAsin)
TOPS_MATH_ENTRY(cosh_forward, kCosh)
TOPS_MATH_ENTRY(sinh_forward, kSinh)
TOPS_MATH_ENTRY(asinh_forward, kAsinh)
TOPS_MATH_ENTRY(acosh_forward, kAcosh)
TOPS_MATH_ENTRY(atanh_forward, kAtanh)
TOPS_MATH_ENTRY(round_forward, kRound)
TOPS_MATH_ENTRY(erf_forward, kErf)
TOPS_MATH_ENTRY(gelu_forward, kGelu)
#undef TOPS_MATH_ENTRY
