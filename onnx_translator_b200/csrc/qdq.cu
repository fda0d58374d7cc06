// QuantizeLinear / DequantizeLinear (tensor_ops.c:999-1034), per tensor and per axis.
//
// The reference reads X, scale and zero point at the same flat index, so its caller materialises
// scale and zero point at full size.  Here they are broadcast operands: a scalar, a [1,C,1,1]
// tensor or a full-size tensor all take the same kernel, and only X and Y stream through HBM.
#include "qdq_bodies.cuh"

namespace tops {

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

bool qdq_fast(const char* name, bool quantize, const Tensor* x, const Tensor* s, const Tensor* z, Tensor* y, const ShapeView& s_shape,
              const ShapeView& z_shape);     // qdq_fast.cu

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

    // float32 against 8-bit codes with one scale, or one per element of the last dimension: the dedicated loops
    bool done = qdq_fast(name, QUANTIZE, x, s, z, y, sv, zv);
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
