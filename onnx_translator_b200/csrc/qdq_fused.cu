// Quantize / Dequantize fused with their elementwise neighbours (tensor_ops.c:999-1034 with :864-997 and
// :708-728 in between): the chains a QDQ graph is full of, evaluated in registers.
//
//   tops_quantize_dequantize_forward   y = DequantizeLinear(QuantizeLinear(x, s, z), s, z)
//       the "fake quantisation" round trip: 4 + 4 bytes per element instead of 5 + 5 (the codes are written too
//       only if the caller wants them: 9 bytes).
//   tops_dq_add_q_forward              y = QuantizeLinear([Relu](DequantizeLinear(a) + DequantizeLinear(b)))
//       the tail of a quantised residual block: 1 + 1 + 1 bytes per element instead of 5 + 5 + 12 [+ 8] + 5.
//
// Both are bit-identical to the chain of separate operators: every intermediate value is rounded to float32
// exactly where the chain would store it (the bodies below are the chain's own arithmetic, qdq_bodies.cuh).
#include "qdq_bodies.cuh"

namespace tops {

// ---- Q -> DQ ----------------------------------------------------------------------------------------------------
template <int DX, int DZ, int DQ, int DO, bool ALIGNED>
struct RoundTripBody {
    using Q = QuantizeBody<DX, DTYPE_FLOAT32, DZ, DQ, ALIGNED>;
    static constexpr int kV = Q::kV;
    static constexpr int kGroups = 0;
    using D = DequantizeBodyN<DQ, DTYPE_FLOAT32, DZ, DO, ALIGNED, kV>;
    Q q;                  // geometry, x, scale, zero point; q.out = where the codes go (null: nowhere)
    void* y;
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        typename Q::Regs r;
        q.load(i0, nv, r);
        typename Q::Codes codes;
        q.compute(r, codes);
        if (q.out) put3<DQ, kV, ALIGNED>(q.out, i0, nv, codes);
        const D d{q.g, q.x, q.s, q.z, y};
        typename D::Values values;
        d.compute(codes, r.rs, r.rz, nv == (uint32_t)kV, values);
        put3<DO, kV, ALIGNED>(y, i0, nv, values);
    }
};

template <int DZ, int DQ>
static bool round_trip_typed(const char* name, const Geometry& geom, Operand* ops, Tensor* codes, Tensor* y) {
    constexpr int DX = DTYPE_FLOAT32, DO = DTYPE_FLOAT32;
    const int bytes[3] = {4, 4, dtype_bytes(DZ)};
    char* code_base = codes ? (char*)codes->data : nullptr;
    return for_each_slab(name, geom, ops, bytes, 3, y->data, 4, y->size, [&](const Slab& s) {
        if (!s.fits3) return false;
        const size_t first = (size_t)((char*)s.out - (char*)y->data) / 4;        // element offset of this slab
        void* slab_codes = code_base ? code_base + first : nullptr;
        constexpr int V = RoundTripBody<DX, DZ, DQ, DO, true>::kV;
        if (slab_aligned(s, 3, bytes, 4, V) && (!slab_codes || aligned_to(slab_codes, 16))) {
            RoundTripBody<DX, DZ, DQ, DO, true> b{{s.geo3, s.ops3[0], s.ops3[1], s.ops3[2], slab_codes}, s.out};
            return launch_body(name, b, s.n);
        }
        RoundTripBody<DX, DZ, DQ, DO, false> b{{s.geo3, s.ops3[0], s.ops3[1], s.ops3[2], slab_codes}, s.out};
        return launch_body(name, b, s.n);
    });
}

// ---- DQ, DQ -> Add [-> Relu] -> Q ----------------------------------------------------------------------------------
template <int DA, int DB, int DO, bool ALIGNED>
struct DqAddQBody {
    static constexpr int kV = 16;
    static constexpr int kGroups = 0;
    const void *a, *b;
    void* out;
    const float *a_scale, *b_scale, *y_scale;
    const void *a_zero, *b_zero, *y_zero;              // one value of the code type each, or null for 0
    int relu;
    template <int DT> static __device__ __forceinline__ float zero_of(const void* p) {
        if (!p) return 0.0f;
        return DT == DTYPE_INT8 ? (float)*(const int8_t*)p : (float)*(const uint8_t*)p;
    }
    __device__ __forceinline__ void operator()(uint32_t i0, uint32_t nv) const {
        using SA = typename Storage<DA>::type;
        using SB = typename Storage<DB>::type;
        Run<SA, kV> ra;
        Run<SB, kV> rb;
        if (ALIGNED && nv == kV) {
            load_bytes_stream<kV>((const SA*)a + i0, &ra);
            load_bytes_stream<kV>((const SB*)b + i0, &rb);
        } else {
            #pragma unroll
            for (int j = 0; j < kV; j++) {
                ra.v[j] = (uint32_t)j < nv ? ((const SA*)a)[i0 + j] : SA(0);
                rb.v[j] = (uint32_t)j < nv ? ((const SB*)b)[i0 + j] : SB(0);
            }
        }
        float fa[kV], fb[kV];
        decode_floats<DA, kV>(ra, fa);
        decode_floats<DB, kV>(rb, fb);
        const float sa = __ldg(a_scale), sb = __ldg(b_scale), sy = __ldg(y_scale);
        const float za = zero_of<DA>(a_zero), zb = zero_of<DB>(b_zero), zy = zero_of<DO>(y_zero);
        const float inv = quantize_reciprocal(sy);
        const int zm = (int)zy - 0x4B400000;
        float sum[kV];
        int v[kV];
        bool all_ok = true;
        #pragma unroll
        for (int j = 0; j < kV; j++) {
            // DequantizeLinear twice: an exact difference and one rounded multiply each; Add: one rounded sum
            const float da = __fmul_rn(__fsub_rn(fa[j], za), sa);
            const float db = __fmul_rn(__fsub_rn(fb[j], zb), sb);
            float t = __fadd_rn(da, db);
            if (relu) t = t > 0.0f ? t : 0.0f;
            sum[j] = t;
            bool ok;
            v[j] = quantize_round_8bit(t, inv, zm, ok);
            all_ok = all_ok & ok;
        }
        Run<typename Storage<DO>::type, kV> ro;
        if (all_ok) {
            encode_ints<DO, kV>(v, ro);
        } else {
            #pragma unroll
            for (int j = 0; j < kV; j++) ro.v[j] = quantize_exact<DO>((double)sum[j], (double)sy, (double)zy);
        }
        put3<DO, kV, ALIGNED>(out, i0, nv, ro);
    }
};

template <int DA, int DB, int DO>
static bool dq_add_q_typed(const char* name, const Tensor* a, const Tensor* b, Tensor* y, const float* sa, const float* sb, const float* sy,
                           const void* za, const void* zb, const void* zy, int relu) {
    const size_t kSlab = 0x7FFFFF00ull;
    bool ok = true;
    for (size_t first = 0; first < y->size && ok; first += kSlab) {
        const size_t n = y->size - first < kSlab ? y->size - first : kSlab;
        const void *pa = (const char*)a->data + first, *pb = (const char*)b->data + first;
        void* po = (char*)y->data + first;
        if (aligned_to(pa, 16) && aligned_to(pb, 16) && aligned_to(po, 16)) {
            DqAddQBody<DA, DB, DO, true> body{pa, pb, po, sa, sb, sy, za, zb, zy, relu};
            ok = launch_body(name, body, n);
        } else {
            DqAddQBody<DA, DB, DO, false> body{pa, pb, po, sa, sb, sy, za, zb, zy, relu};
            ok = launch_body(name, body, n);
        }
    }
    return ok;
}

static bool code8(int dt) { return dt == DTYPE_INT8 || dt == DTYPE_UINT8; }
static bool one_scale(const Tensor* t) { return t && t->data && t->dtype == DTYPE_FLOAT32 && t->size == 1; }
static bool one_zero(const Tensor* t, int dt) { return !t || !t->data || ((int)t->dtype == dt && t->size == 1); }

static int refuse(const char* name, int code, const char* what, Tensor* y, Tensor* y2 = nullptr) {
    set_error(code, "%s: %s", name, what);
    zero_fill(y);
    zero_fill(y2);
    return tops_last_error();
}

}  // namespace tops

using namespace tops;

TOPS_API int tops_quantize_dequantize_forward(const Tensor* X, const Tensor* Scale, const Tensor* ZeroPoint, Tensor* Codes, Tensor* Y) {
    const char* name = "tops_quantize_dequantize_forward";
    if (!X || !Scale || !ZeroPoint || !Y || !X->data || !Scale->data || !ZeroPoint->data || !Y->data || (Codes && !Codes->data))
        return refuse(name, TOPS_ERR_INVALID, "null tensor", Y, Codes);
    if (X->size != Y->size || (Codes && Codes->size != Y->size))
        return refuse(name, TOPS_ERR_INVALID, "X, the codes and Y must have one element count", Y, Codes);
    const int dz = (int)ZeroPoint->dtype;
    const int dq = Codes ? (int)Codes->dtype : dz;                  // without a codes tensor the zero point's type is the code type
    if (X->dtype != DTYPE_FLOAT32 || Y->dtype != DTYPE_FLOAT32 || Scale->dtype != DTYPE_FLOAT32)
        return refuse(name, TOPS_ERR_UNSUPPORTED, "covers float32 X, Scale and Y", Y, Codes);
    Geometry geom;
    Operand ops[3];
    const ShapeView out{Y->shape, Y->ndim, Y->size};
    const ShapeView ins[3] = {{X->shape, X->ndim, X->size}, {Scale->shape, Scale->ndim, Scale->size}, {ZeroPoint->shape, ZeroPoint->ndim, ZeroPoint->size}};
    if (!plan_broadcast(out, ins, 3, &geom, ops))
        return refuse(name, TOPS_ERR_INVALID, "scale / zero point do not broadcast to X's shape", Y, Codes);
    ops[0].ptr = X->data; ops[1].ptr = Scale->data; ops[2].ptr = ZeroPoint->data;
    if (Y->size == 0) return TOPS_OK;
    bool done = false, ok = false;
#define TOPS_RT(Z, Q) if (!done && dz == Z && dq == Q) { ok = round_trip_typed<Z, Q>(name, geom, ops, Codes, Y); done = true; }
    TOPS_RT(DTYPE_INT8, DTYPE_INT8) TOPS_RT(DTYPE_UINT8, DTYPE_UINT8)
    TOPS_RT(DTYPE_FLOAT8_E4M3, DTYPE_FLOAT8_E4M3) TOPS_RT(DTYPE_FLOAT8_E5M2, DTYPE_FLOAT8_E5M2)
    TOPS_RT(DTYPE_INT8, DTYPE_FLOAT8_E4M3) TOPS_RT(DTYPE_INT8, DTYPE_FLOAT8_E5M2)
#undef TOPS_RT
    if (!done) return refuse(name, TOPS_ERR_UNSUPPORTED, "covers int8 / uint8 / float8 codes with a zero point of the code type (or int8 for float8)", Y, Codes);
    if (!ok) {
        if (tops_last_error() == TOPS_OK) return refuse(name, TOPS_ERR_UNSUPPORTED, "broadcast pattern with more than three levels", Y, Codes);
        return tops_last_error();
    }
    finish_op();
    return TOPS_OK;
}

TOPS_API int tops_dq_add_q_forward(const Tensor* A, const Tensor* a_scale, const Tensor* a_zero, const Tensor* B, const Tensor* b_scale,
                                   const Tensor* b_zero, const Tensor* y_scale, const Tensor* y_zero, Tensor* Y, int relu) {
    const char* name = "tops_dq_add_q_forward";
    if (!A || !B || !Y || !A->data || !B->data || !Y->data) return refuse(name, TOPS_ERR_INVALID, "null tensor", Y);
    if (A->size != Y->size || B->size != Y->size) return refuse(name, TOPS_ERR_UNSUPPORTED, "A, B and Y must have one element count (no broadcasting)", Y);
    const int da = (int)A->dtype, db = (int)B->dtype, dy = (int)Y->dtype;
    if (!code8(da) || !code8(db) || !code8(dy) || !one_scale(a_scale) || !one_scale(b_scale) || !one_scale(y_scale) ||
        !one_zero(a_zero, da) || !one_zero(b_zero, db) || !one_zero(y_zero, dy))
        return refuse(name, TOPS_ERR_UNSUPPORTED, "covers int8 / uint8 codes with one float32 scale and one zero point of the code type per tensor", Y);
    if (Y->size == 0) return TOPS_OK;
    if (!acquire_device()) return tops_last_error();
    const float *sa = (const float*)a_scale->data, *sb = (const float*)b_scale->data, *sy = (const float*)y_scale->data;
    const void *za = (a_zero && a_zero->data) ? a_zero->data : nullptr, *zb = (b_zero && b_zero->data) ? b_zero->data : nullptr;
    const void* zy = (y_zero && y_zero->data) ? y_zero->data : nullptr;
    bool ok = false;
#define TOPS_DAQ(TA, TB, TO) if (da == TA && db == TB && dy == TO) ok = dq_add_q_typed<TA, TB, TO>(name, A, B, Y, sa, sb, sy, za, zb, zy, relu ? 1 : 0);
    TOPS_DAQ(DTYPE_INT8, DTYPE_INT8, DTYPE_INT8) TOPS_DAQ(DTYPE_INT8, DTYPE_INT8, DTYPE_UINT8)
    TOPS_DAQ(DTYPE_INT8, DTYPE_UINT8, DTYPE_INT8) TOPS_DAQ(DTYPE_INT8, DTYPE_UINT8, DTYPE_UINT8)
    TOPS_DAQ(DTYPE_UINT8, DTYPE_INT8, DTYPE_INT8) TOPS_DAQ(DTYPE_UINT8, DTYPE_INT8, DTYPE_UINT8)
    TOPS_DAQ(DTYPE_UINT8, DTYPE_UINT8, DTYPE_INT8) TOPS_DAQ(DTYPE_UINT8, DTYPE_UINT8, DTYPE_UINT8)
#undef TOPS_DAQ
    if (!ok) return tops_last_error();
    finish_op();
    return TOPS_OK;
}
