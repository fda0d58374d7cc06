// QuantizeLinear / DequantizeLinear (tensor_ops.c:999-1034), per tensor and per axis.
//
// The reference reads X, scale and zero point at the same flat index, so its caller materialises
// scale and zero point at full size.  Here they are broadcast operands: a scalar, a [1,C,1,1]
// tensor or a full-size tensor all take the same kernel, and only X and Y stream through HBM.
#include "elementwise.cuh"
#include "qdq_math.cuh"

namespace tops {

// ---- Quantize (arithmetic: qdq_math.cuh) -------------------------------------------------------------
template <int DX, int DS, int DZ, int DO, bool ALIGNED>
struct QuantizeBody {
    static constexpr int kV = vec_width(dtype_bytes(DX), dtype_bytes(DO), dtype_bytes(DO), 64);
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
        const Run<typename Storage<DX>::type, kV>& rx = r.rx;
        const Run<typename Storage<DS>::type, kV>& rs = r.rs;
        const Run<typename Storage<DZ>::type, kV>& rz = r.rz;
        Run<typename Storage<DO>::type, kV> ro;
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
                    put3<DO, kV, ALIGNED>(out, i0, nv, ro);
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
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
};

// ---- Dequantize ----------------------------------------------------------------------------------------
// Reference arithmetic: (x - z) * s in double, rounded once on store.  In float32 the same bits
// come out whenever x - z is exact in float32 (8-bit integers, e4m3 codes, any x with z == 0):
// the double product of a <= 24-bit difference and a 24-bit scale is exact, so a single
// correctly rounded float multiply reproduces "exact product, one rounding".
template <int DX, int DS, int DZ, int DO, bool ALIGNED>
struct DequantizeBody {
    static constexpr bool kDiffExact = dtype_exact_in_f32(DX) && dtype_exact_in_f32(DZ) && dtype_exact_in_f32(DS) &&
        DX != DTYPE_FLOAT8_E5M2 && DZ != DTYPE_FLOAT8_E5M2 && DX != DTYPE_FLOAT16 && DZ != DTYPE_FLOAT16 &&
        DX != DTYPE_BFLOAT16 && DZ != DTYPE_BFLOAT16 && DX != DTYPE_FLOAT32 && DZ != DTYPE_FLOAT32 &&
        DO != DTYPE_FLOAT64 && !dtype_is_int(DO);
    static constexpr int kV = vec_width(dtype_bytes(DX), dtype_bytes(DO), dtype_bytes(DO));
    static constexpr int kGroups = 2;
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
        const Run<typename Storage<DX>::type, kV>& rx = r.rx;
        const Run<typename Storage<DS>::type, kV>& rs = r.rs;
        const Run<typename Storage<DZ>::type, kV>& rz = r.rz;
        Run<typename Storage<DO>::type, kV> ro;
        if constexpr (kDiffExact && (DX == DTYPE_INT8 || DX == DTYPE_UINT8) && kV % 4 == 0) {
            // one scale and one zero point for the whole run: the byte is placed in the low mantissa
            // byte of 2^23 and (2^23 + offset + z) is subtracted in one exact step
            if (ALIGNED && nv == kV && !g.simple && s.st2 == 0 && z.st2 == 0) {
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
                put3<DO, kV, ALIGNED>(out, i0, nv, ro);
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
            put3<DO, kV, ALIGNED>(out, i0, nv, ro);
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
                put3<DO, kV, ALIGNED>(out, i0, nv, ro);
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
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
};

// ---- any dtype combination -------------------------------------------------------------------------------
template <bool QUANTIZE>
struct QdqGenericBody {
    static constexpr int kV = 1;
    static constexpr int kGroups = 0;
    Geometry g;
    Operand x, s, z;
    void* out;
    int dx, ds, dz, dout;
    __device__ __forceinline__ void operator()(uint32_t i, uint32_t) const {
        uint32_t p;
        const double xv = load_f64_rt(x.ptr, dx, x.flat ? i : operand_offset(g, x, i, p));
        const double sv = load_f64_rt(s.ptr, ds, s.flat ? i : operand_offset(g, s, i, p));
        const double zv = load_f64_rt(z.ptr, dz, z.flat ? i : operand_offset(g, z, i, p));
        double r;
        if constexpr (QUANTIZE) { r = zv; if (sv != 0.0) r = __dadd_rn(rint(__ddiv_rn(xv, sv)), zv); }
        else r = __dmul_rn(__dsub_rn(xv, zv), sv);
        store_f64_rt(out, dout, i, r);
    }
};

template <bool QUANTIZE>
static bool qdq_generic_slab(const char* name, const Slab& s, int dx, int ds, int dz, int dout) {
    QdqGenericBody<QUANTIZE> b{s.geom, s.ops[0], s.ops[1], s.ops[2], s.out, dx, ds, dz, dout};
    return launch_body(name, b, s.n);
}

template <template <int, int, int, int, bool> class Body, bool QUANTIZE, int DX, int DS, int DZ, int DO>
static bool qdq_typed(const char* name, const Geometry& geom, Operand* ops, Tensor* y) {
    const int bytes[3] = {dtype_bytes(DX), dtype_bytes(DS), dtype_bytes(DZ)};
    return for_each_slab(name, geom, ops, bytes, 3, y->data, dtype_bytes(DO), y->size, [&](const Slab& s) {
        if (!s.fits3) return qdq_generic_slab<QUANTIZE>(name, s, DX, DS, DZ, DO);
        constexpr int V = Body<DX, DS, DZ, DO, true>::kV;
        if (slab_aligned(s, 3, bytes, dtype_bytes(DO), V)) {
            Body<DX, DS, DZ, DO, true> b{s.geo3, s.ops3[0], s.ops3[1], s.ops3[2], s.out};
            return launch_body(name, b, s.n);
        }
        Body<DX, DS, DZ, DO, false> b{s.geo3, s.ops3[0], s.ops3[1], s.ops3[2], s.out};
        return launch_body(name, b, s.n);
    });
}

// axis >= 0: Scale / ZeroPoint are 1-D of length Y.shape[axis]; axis < -64: plain broadcasting.
constexpr int kNoAxis = -1000;

template <bool QUANTIZE>
static void qdq_forward(const char* name, const Tensor* x, const Tensor* s, const Tensor* z, Tensor* y, int axis) {
    if (!x || !s || !z || !y || !x->data || !s->data || !z->data || !y->data) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor", name);
        zero_fill(y);
        return;
    }
    const int dx = (int)x->dtype, ds = (int)s->dtype, dz = (int)z->dtype, dout = (int)y->dtype;
    if (!dtype_valid(dx) || !dtype_valid(ds) || !dtype_valid(dz) || !dtype_valid(dout)) { set_error(TOPS_ERR_INVALID, "%s: bad dtype", name); return; }

    int axis_shape[16];
    ShapeView sv{s->shape, s->ndim, s->size}, zv{z->shape, z->ndim, z->size};
    if (axis != kNoAxis) {
        const int nd = y->ndim;
        if (axis < 0) axis += nd;
        if (nd > 16 || axis < 0 || axis >= nd || s->size != (size_t)y->shape[axis] || (z->size != s->size && z->size != 1)) {
            set_error(TOPS_ERR_INVALID, "%s: scale length does not match the axis", name);
            zero_fill(y);
            return;
        }
        for (int d = 0; d < nd; d++) axis_shape[d] = 1;
        axis_shape[axis] = y->shape[axis];
        sv = ShapeView{axis_shape, nd, s->size};
        if (z->size == s->size) zv = ShapeView{axis_shape, nd, z->size};
    }
    Geometry geom;
    Operand ops[3];
    const ShapeView out{y->shape, y->ndim, y->size};
    const ShapeView ins[3] = {{x->shape, x->ndim, x->size}, sv, zv};
    if (!plan_broadcast(out, ins, 3, &geom, ops)) {
        set_error(TOPS_ERR_INVALID, "%s: operand shapes do not broadcast to the output shape", name);
        zero_fill(y);
        return;
    }
    ops[0].ptr = x->data; ops[1].ptr = s->data; ops[2].ptr = z->data;

    bool done = false;
#define TOPS_Q(X, Z, O) if (!done && dx == X && ds == DTYPE_FLOAT32 && dz == Z && dout == O) { \
        qdq_typed<QuantizeBody, true, X, DTYPE_FLOAT32, Z, O>(name, geom, ops, y); done = true; }
#define TOPS_DQ(X, Z, O) if (!done && dx == X && ds == DTYPE_FLOAT32 && dz == Z && dout == O) { \
        qdq_typed<DequantizeBody, false, X, DTYPE_FLOAT32, Z, O>(name, geom, ops, y); done = true; }
    if (QUANTIZE) {
#define TOPS_Q_SOURCES(Z, O) TOPS_Q(DTYPE_FLOAT32, Z, O) TOPS_Q(DTYPE_FLOAT16, Z, O) TOPS_Q(DTYPE_BFLOAT16, Z, O)
        TOPS_Q_SOURCES(DTYPE_INT8, DTYPE_INT8) TOPS_Q_SOURCES(DTYPE_UINT8, DTYPE_UINT8)
        TOPS_Q_SOURCES(DTYPE_FLOAT8_E4M3, DTYPE_FLOAT8_E4M3) TOPS_Q_SOURCES(DTYPE_FLOAT8_E5M2, DTYPE_FLOAT8_E5M2)
        TOPS_Q_SOURCES(DTYPE_INT8, DTYPE_FLOAT8_E4M3) TOPS_Q_SOURCES(DTYPE_INT8, DTYPE_FLOAT8_E5M2)
#undef TOPS_Q_SOURCES
    } else {
#define TOPS_DQ_TARGETS(X, Z) TOPS_DQ(X, Z, DTYPE_FLOAT32) TOPS_DQ(X, Z, DTYPE_FLOAT16) TOPS_DQ(X, Z, DTYPE_BFLOAT16)
        TOPS_DQ_TARGETS(DTYPE_INT8, DTYPE_INT8) TOPS_DQ_TARGETS(DTYPE_UINT8, DTYPE_UINT8)
        TOPS_DQ_TARGETS(DTYPE_FLOAT8_E4M3, DTYPE_FLOAT8_E4M3) TOPS_DQ_TARGETS(DTYPE_FLOAT8_E5M2, DTYPE_FLOAT8_E5M2)
        TOPS_DQ_TARGETS(DTYPE_FLOAT8_E4M3, DTYPE_INT8) TOPS_DQ_TARGETS(DTYPE_FLOAT8_E5M2, DTYPE_INT8)
        TOPS_DQ_TARGETS(DTYPE_INT32, DTYPE_INT32)
#undef TOPS_DQ_TARGETS
    }
#undef TOPS_Q
#undef TOPS_DQ
    if (!done) {
        const int bytes[3] = {dtype_bytes(dx), dtype_bytes(ds), dtype_bytes(dz)};
        for_each_slab(name, geom, ops, bytes, 3, y->data, dtype_bytes(dout), y->size,
                      [&](const Slab& s) { return qdq_generic_slab<QUANTIZE>(name, s, dx, ds, dz, dout); });
    }
    finish_op();
}

}  // namespace tops

using namespace tops;

TOPS_API void quantize_linear_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y) {
    qdq_forward<true>("quantize_linear_forward", X, Scale, ZeroPoint, Y, kNoAxis);
}
TOPS_API void dequantize_linear_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y) {
    qdq_forward<false>("dequantize_linear_forward", X, Scale, ZeroPoint, Y, kNoAxis);
}
TOPS_API void tops_quantize_linear_axis_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y, int axis) {
    qdq_forward<true>("tops_quantize_linear_axis_forward", X, Scale, ZeroPoint, Y, axis);
}
TOPS_API void tops_dequantize_linear_axis_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Y, int axis) {
    qdq_forward<false>("tops_dequantize_linear_axis_forward", X, Scale, ZeroPoint, Y, axis);
}
