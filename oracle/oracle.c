/*
 * oracle.c -- CPU restatement of the reference operator library's hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker the parity tests hold the CUDA library
 * against; nothing in the product imports, links or executes it.  It restates, in independent
 * code, the arithmetic of Sakauma/onnx_translator's tensor_ops/tensor_ops.c for the 13 hot-path
 * operators plus the dtype codecs.  Every function cites the reference lines it follows.
 *
 * Parity pin: tests/test_oracle_pin.py runs this library against the reference's own
 * tensor_ops.c compiled unchanged (oracle/_ref/tensor_ops_ref.so, see oracle/Makefile) on seeded
 * inputs, and against the golden vectors under tests/golden/ that were generated from that same
 * compiled reference (tests/golden/make_golden.py).
 *
 * Conventions shared with the reference (tensor_ops/tensor_ops.h:10-34): the dtype codes, the
 * Tensor struct layout, dense row-major data, int4 stored one value per byte.
 */
#include <float.h>
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* tensor_ops/tensor_ops.h:10-23 */
enum {
    DT_E4M3 = 0, DT_E5M2 = 1, DT_F16 = 2, DT_BF16 = 3, DT_F32 = 4, DT_F64 = 5,
    DT_I4 = 6, DT_I8 = 7, DT_U8 = 8, DT_I16 = 9, DT_I32 = 10, DT_I64 = 11
};

/* tensor_ops/tensor_ops.h:28-34 */
typedef struct {
    void*  data;
    int*   shape;
    int    ndim;
    size_t size;
    int    dtype;
} OrcTensor;

/* tensor_ops/tensor_ops.h:39-54 */
typedef struct { int* pads; int* strides; int* dilations; int group; } OrcConvParams;
typedef struct { int* pads; int* strides; int* dilations; int* kernel_shape; } OrcPoolParams;

static const int k_elem_bytes[12] = {1, 1, 2, 2, 4, 8, 1, 1, 1, 2, 4, 8};

static int is_integer_dtype(int dt) { return dt >= DT_I4 && dt <= DT_I64; }

ORC_API size_t orc_dtype_size(int dt) { return (dt >= 0 && dt < 12) ? (size_t)k_elem_bytes[dt] : 4; }

/* ------------------------------------------------------------------------------------------
 * Small-float codecs.  One parametric decoder/encoder serves fp16, e4m3 and e5m2; the format
 * table carries what distinguishes the reference's encoders from IEEE:
 *   fp16  (tensor_ops.c:104-152): RNE with subnormal outputs, but anything below 2^-24 -> +-0;
 *                                 overflow -> Inf; NaN -> sign|0x7FFF.
 *   e4m3  (tensor_ops.c:258-287): no subnormal outputs (|x| < 2^-6 -> +-0); overflow, Inf and a
 *                                 round-up into the NaN code saturate to 0x7E; NaN -> 0x7F|sign.
 *   e5m2  (tensor_ops.c:318-347): |x| < 2^-14 -> +-0; overflow -> Inf 0x7C; NaN -> 0x7D|sign.
 * Decoders (tensor_ops.c:160-184, 236-256, 295-316) are plain: subnormals are honoured.
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    int ebits, mbits, bias;
    int flush_below_exp;   /* inputs with unbiased exponent below this become signed zero   */
    int ieee_specials;     /* 1: top exponent is Inf/NaN; 0: only all-ones is NaN (e4m3fn)   */
    int saturate;          /* 1: overflow clamps to the largest finite code                  */
    uint32_t nan_code;     /* magnitude bits written for a NaN input                         */
} MiniFmt;

static const MiniFmt FMT_F16  = {5, 10, 15, -24, 1, 0, 0x7FFFu};
static const MiniFmt FMT_E4M3 = {4,  3,  7,  -6, 0, 1, 0x7Fu};
static const MiniFmt FMT_E5M2 = {5,  2, 15, -14, 1, 0, 0x7Du};

static float f32_from_bits(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t bits_from_f32(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

static float mini_decode(uint32_t code, const MiniFmt* F) {
    const int total = 1 + F->ebits + F->mbits;
    const uint32_t sign = (code >> (total - 1)) & 1u;
    const uint32_t e = (code >> F->mbits) & ((1u << F->ebits) - 1u);
    const uint32_t m = code & ((1u << F->mbits) - 1u);
    const uint32_t emax = (1u << F->ebits) - 1u;
    const uint32_t s32 = sign << 31;
    if (F->ieee_specials && e == emax) {
        if (m == 0) return f32_from_bits(s32 | 0x7F800000u);
        /* payload keeps its position below the f32 exponent; e5m2 also forces the quiet bit */
        uint32_t payload = m << (23 - F->mbits);
        if (F->mbits == 2) payload |= 0x400000u;
        return f32_from_bits(s32 | 0x7F800000u | payload);
    }
    if (!F->ieee_specials && e == emax && m == (1u << F->mbits) - 1u)
        return f32_from_bits(s32 | 0x7FC00000u);
    float mag;
    if (e == 0) mag = ldexpf((float)m, 1 - F->bias - F->mbits);
    else        mag = ldexpf((float)((1u << F->mbits) | m), (int)e - F->bias - F->mbits);
    return sign ? -mag : mag;
}

static uint32_t mini_encode(float value, const MiniFmt* F) {
    const uint32_t u = bits_from_f32(value);
    const int total = 1 + F->ebits + F->mbits;
    const uint32_t sign = (u >> 31) << (total - 1);
    const uint32_t e32 = (u >> 23) & 0xFFu;
    const uint32_t m32 = u & 0x7FFFFFu;
    const uint32_t emax = (1u << F->ebits) - 1u;
    const uint32_t inf_code = emax << F->mbits;
    const uint32_t max_finite = F->ieee_specials ? (inf_code - 1u)
                                                 : ((emax << F->mbits) | ((1u << F->mbits) - 2u));
    const uint32_t overflow_code = F->saturate ? max_finite : inf_code;

    if (e32 == 255u) {
        if (m32) return sign | F->nan_code;
        return sign | overflow_code;             /* Inf: kept (fp16/e5m2) or saturated (e4m3) */
    }
    if (e32 == 0u) return sign;                    /* f32 zero or subnormal */
    const int unbiased = (int)e32 - 127;
    if (unbiased < F->flush_below_exp) return sign;

    /* Round the 24-bit significand to mbits fraction bits (more are dropped for subnormal
       results), ties to even.  `keep` counts the significand bits that survive. */
    int target_e = unbiased + F->bias;             /* biased exponent in the small format */
    int drop = 23 - F->mbits;
    if (target_e <= 0) { drop += 1 - target_e; target_e = 0; }
    const uint32_t sig = m32 | 0x800000u;
    uint32_t kept = sig >> drop;
    const uint32_t rem = sig & ((1u << drop) - 1u);
    const uint32_t half = 1u << (drop - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    /* kept now holds (implicit bit + fraction) for normals, or the bare fraction for
       subnormals; adding it to the exponent field carries correctly in both cases. */
    uint32_t code;
    if (target_e == 0) code = kept;                                   /* may carry into e=1 */
    else               code = ((uint32_t)(target_e - 1) << F->mbits) + kept;
    if (code > max_finite) return sign | overflow_code;
    return sign | code;
}

/* tensor_ops.c:192-210: RNE on the upper 16 bits; NaN keeps its top payload and gets 0x40. */
static uint16_t bf16_encode(float value) {
    const uint32_t u = bits_from_f32(value);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    const uint32_t rounded = u + 0x7FFFu + ((u >> 16) & 1u);
    return (uint16_t)(rounded >> 16);              /* a carry into the exponent yields Inf */
}
/* tensor_ops.c:218-228 */
static float bf16_decode(uint16_t code) { return f32_from_bits((uint32_t)code << 16); }

ORC_API uint32_t orc_encode(int dt, float v) {
    switch (dt) {
        case DT_E4M3: return mini_encode(v, &FMT_E4M3);
        case DT_E5M2: return mini_encode(v, &FMT_E5M2);
        case DT_F16:  return mini_encode(v, &FMT_F16);
        case DT_BF16: return bf16_encode(v);
        default:      return bits_from_f32(v);
    }
}
ORC_API float orc_decode(int dt, uint32_t code) {
    switch (dt) {
        case DT_E4M3: return mini_decode(code & 0xFFu, &FMT_E4M3);
        case DT_E5M2: return mini_decode(code & 0xFFu, &FMT_E5M2);
        case DT_F16:  return mini_decode(code & 0xFFFFu, &FMT_F16);
        case DT_BF16: return bf16_decode((uint16_t)code);
        default:      return f32_from_bits(code);
    }
}

/* ------------------------------------------------------------------------------------------
 * Element access.  tensor_ops.c:488-546 (loads), 552-588 (stores), 64-96 (saturation).
 * ---------------------------------------------------------------------------------------- */

/* (int64_t)x as the reference's x86-64 build performs it: cvttsd2si returns the "integer
   indefinite" value INT64_MIN for NaN, +-Inf and anything outside [-2^63, 2^63). */
static int64_t trunc_to_i64_x86(double v) {
    if (!(v >= -9223372036854775808.0 && v < 9223372036854775808.0)) return INT64_MIN;
    return (int64_t)v;
}

static int64_t int4_value(int8_t raw) {           /* tensor_ops.c:464-474: low nibble, signed */
    int v = raw & 0x0F;
    return (v & 0x08) ? v - 16 : v;
}

static double load_f64(const OrcTensor* t, size_t i) {
    const void* p = t->data;
    switch (t->dtype) {
        case DT_E4M3: return (double)mini_decode(((const uint8_t*)p)[i], &FMT_E4M3);
        case DT_E5M2: return (double)mini_decode(((const uint8_t*)p)[i], &FMT_E5M2);
        case DT_F16:  return (double)mini_decode(((const uint16_t*)p)[i], &FMT_F16);
        case DT_BF16: return (double)bf16_decode(((const uint16_t*)p)[i]);
        case DT_F32:  return (double)((const float*)p)[i];
        case DT_F64:  return ((const double*)p)[i];
        case DT_I4:   return (double)int4_value(((const int8_t*)p)[i]);
        case DT_I8:   return (double)((const int8_t*)p)[i];
        case DT_U8:   return (double)((const uint8_t*)p)[i];
        case DT_I16:  return (double)((const int16_t*)p)[i];
        case DT_I32:  return (double)((const int32_t*)p)[i];
        case DT_I64:  return (double)((const int64_t*)p)[i];
        default:      return 0.0;
    }
}

/* Float sources are rounded to nearest-even in their own precision first (rintf / rint). */
static int64_t load_i64(const OrcTensor* t, size_t i) {
    const void* p = t->data;
    switch (t->dtype) {
        case DT_E4M3: return trunc_to_i64_x86(rintf(mini_decode(((const uint8_t*)p)[i], &FMT_E4M3)));
        case DT_E5M2: return trunc_to_i64_x86(rintf(mini_decode(((const uint8_t*)p)[i], &FMT_E5M2)));
        case DT_F16:  return trunc_to_i64_x86(rintf(mini_decode(((const uint16_t*)p)[i], &FMT_F16)));
        case DT_BF16: return trunc_to_i64_x86(rintf(bf16_decode(((const uint16_t*)p)[i])));
        case DT_F32:  return trunc_to_i64_x86(rintf(((const float*)p)[i]));
        case DT_F64:  return trunc_to_i64_x86(rint(((const double*)p)[i]));
        case DT_I4:   return int4_value(((const int8_t*)p)[i]);
        case DT_I8:   return ((const int8_t*)p)[i];
        case DT_U8:   return ((const uint8_t*)p)[i];
        case DT_I16:  return ((const int16_t*)p)[i];
        case DT_I32:  return ((const int32_t*)p)[i];
        case DT_I64:  return ((const int64_t*)p)[i];
        default:      return 0;
    }
}

static int64_t clamp_i64(int64_t v, int64_t lo, int64_t hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void store_i64(OrcTensor* t, size_t i, int64_t v) {
    void* p = t->data;
    switch (t->dtype) {
        case DT_I4:   ((int8_t*)p)[i]  = (int8_t)clamp_i64(v, -8, 7); break;
        case DT_I8:   ((int8_t*)p)[i]  = (int8_t)clamp_i64(v, -128, 127); break;
        case DT_U8:   ((uint8_t*)p)[i] = (uint8_t)clamp_i64(v, 0, 255); break;
        case DT_I16:  ((int16_t*)p)[i] = (int16_t)clamp_i64(v, -32768, 32767); break;
        case DT_I32:  ((int32_t*)p)[i] = (int32_t)clamp_i64(v, INT32_MIN, INT32_MAX); break;
        case DT_I64:  ((int64_t*)p)[i] = v; break;
        case DT_E4M3: ((uint8_t*)p)[i]  = (uint8_t)mini_encode((float)v, &FMT_E4M3); break;
        case DT_E5M2: ((uint8_t*)p)[i]  = (uint8_t)mini_encode((float)v, &FMT_E5M2); break;
        case DT_F16:  ((uint16_t*)p)[i] = (uint16_t)mini_encode((float)v, &FMT_F16); break;
        case DT_BF16: ((uint16_t*)p)[i] = bf16_encode((float)v); break;
        case DT_F32:  ((float*)p)[i]  = (float)v; break;
        case DT_F64:  ((double*)p)[i] = (double)v; break;
        default: break;
    }
}

static void store_f64(OrcTensor* t, size_t i, double v) {
    void* p = t->data;
    switch (t->dtype) {
        case DT_E4M3: ((uint8_t*)p)[i]  = (uint8_t)mini_encode((float)v, &FMT_E4M3); break;
        case DT_E5M2: ((uint8_t*)p)[i]  = (uint8_t)mini_encode((float)v, &FMT_E5M2); break;
        case DT_F16:  ((uint16_t*)p)[i] = (uint16_t)mini_encode((float)v, &FMT_F16); break;
        case DT_BF16: ((uint16_t*)p)[i] = bf16_encode((float)v); break;
        case DT_F32:  ((float*)p)[i]  = (float)v; break;
        case DT_F64:  ((double*)p)[i] = v; break;
        default:      /* integer targets: nearest-even, then the saturating integer store */
            if (is_integer_dtype(t->dtype)) store_i64(t, i, trunc_to_i64_x86(rint(v)));
            break;
    }
}

/* ------------------------------------------------------------------------------------------
 * Unary operators.
 * ---------------------------------------------------------------------------------------- */

static int unary_args_ok(const OrcTensor* x, const OrcTensor* y) {
    return x && y && x->data && y->data && x->size == y->size;
}

/* tensor_ops.c:708-728: the branch is taken on the INPUT dtype; the float path maps NaN and
   -0 to +0 because the test is `v > 0`. */
ORC_API void orc_relu(const OrcTensor* x, OrcTensor* y) {
    if (!unary_args_ok(x, y)) return;
    const int as_int = is_integer_dtype(x->dtype);
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) {
        if (as_int) { int64_t v = load_i64(x, i); store_i64(y, i, v > 0 ? v : 0); }
        else        { double v = load_f64(x, i);  store_f64(y, i, v > 0 ? v : 0.0); }
    }
}

/* tensor_ops.c:736-757 */
ORC_API void orc_abs(const OrcTensor* x, OrcTensor* y) {
    if (!unary_args_ok(x, y)) return;
    const int as_int = is_integer_dtype(x->dtype);
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) {
        if (as_int) {
            int64_t v = load_i64(x, i);
            store_i64(y, i, v == INT64_MIN ? INT64_MAX : (v < 0 ? -v : v));
        } else {
            store_f64(y, i, fabs(load_f64(x, i)));
        }
    }
}

/* Cosine by table.  tensor_ops.c:17-31 (constants), 763-807 (table), 815-833 (lookup). */
#define LUT_N 4096
static const double kPi = 3.141592653589793238462643383279502884197;
static double g_cos_table[LUT_N + 1];
static int g_cos_table_ready = 0;

ORC_API void orc_init_cos_lut(void) {
    #pragma omp critical(orc_cos_table)
    {
        if (!g_cos_table_ready) {
            const double two_pi = 2.0 * kPi, half_pi = kPi / 2.0;
            for (int i = 0; i <= LUT_N; i++) {
                double a = (double)i * two_pi / LUT_N;      /* angle in [0, 2pi] */
                double sgn = 1.0;
                if (a > kPi) a = two_pi - a;                /* fold to [0, pi]   */
                if (a > half_pi) { a = kPi - a; sgn = -1.0; } /* fold to [0, pi/2] */
                double r;
                if (a < 0.785398163397448) {                /* cosine series, degree 8 */
                    const double q = a * a;
                    r = 1.0 + q * (-0.5 + q * (0.04166666666666666 +
                        q * (-0.001388888888888889 + q * 0.000024801587301587302)));
                } else {                                    /* sine series of (pi/2 - a), degree 9 */
                    const double t = half_pi - a, q = t * t;
                    r = t * (1.0 + q * (-0.16666666666666666 + q * (0.008333333333333333 +
                        q * (-0.0001984126984126984 + q * 0.0000027557319223985893))));
                }
                g_cos_table[i] = sgn * r;
            }
            g_cos_table_ready = 1;
        }
    }
}

ORC_API const double* orc_cos_table(void) { orc_init_cos_lut(); return g_cos_table; }

static double cos_by_table(double x) {
    const double two_pi = 2.0 * kPi;
    const double r = fmod(fabs(x), two_pi);
    const double pos = r * LUT_N / two_pi;                  /* multiply, then divide */
    int k = (int)pos;
    double w = pos - k;
    if (k >= LUT_N) { k = LUT_N - 1; w = 0.0; }
    return g_cos_table[k] * (1.0 - w) + g_cos_table[k + 1] * w;
}

/* tensor_ops.c:840-854.  NaN/Inf inputs index out of bounds in the reference (undefined);
   here they produce NaN so the checker never faults -- such inputs are outside parity. */
ORC_API void orc_cos(const OrcTensor* x, OrcTensor* y) {
    if (!unary_args_ok(x, y)) return;
    orc_init_cos_lut();
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) {
        const double v = load_f64(x, i);
        store_f64(y, i, isfinite(v) ? cos_by_table(v) : NAN);
    }
}

/* ------------------------------------------------------------------------------------------
 * Binary operators.  tensor_ops.c:610-684 (integer outputs), 864-997 (dispatch).
 * Operands must already have the output's size; broadcasting is the caller's job
 * (nn/__init__.py:210-248).
 * ---------------------------------------------------------------------------------------- */
enum { OP_ADD = 0, OP_SUB = 1, OP_MUL = 2, OP_DIV = 3, OP_MAX = 4, OP_MIN = 5 };

/* int64 arithmetic wraps (the reference relies on two's-complement behaviour at -O3). */
static int64_t int_binary(int op, int64_t a, int64_t b) {
    switch (op) {
        case OP_ADD: return (int64_t)((uint64_t)a + (uint64_t)b);
        case OP_SUB: return (int64_t)((uint64_t)a - (uint64_t)b);
        case OP_MUL: return (int64_t)((uint64_t)a * (uint64_t)b);
        case OP_MAX: return a > b ? a : b;                      /* tensor_ops.c:1351-1352 */
        case OP_MIN: return a < b ? a : b;
        default:
            if (b == 0) return a >= 0 ? INT64_MAX : INT64_MIN;   /* tensor_ops.c:684 */
            if (a == INT64_MIN && b == -1) return INT64_MIN;     /* idiv would trap; keep wrap */
            return a / b;
    }
}

static double float_binary(int op, double a, double b) {
    switch (op) {
        case OP_ADD: return a + b;
        case OP_SUB: return a - b;
        case OP_MUL: return a * b;
        case OP_MAX: return a > b ? a : b;                      /* a NaN on either side yields b */
        case OP_MIN: return a < b ? a : b;
        default:     return a / b;
    }
}

static void binary_forward(int op, const OrcTensor* a, const OrcTensor* b, OrcTensor* o) {
    if (!a || !b || !o || !a->data || !b->data || !o->data) return;
    if (a->size != b->size || a->size != o->size) return;
    if (is_integer_dtype(o->dtype)) {
        #pragma omp parallel for
        for (size_t i = 0; i < o->size; i++)
            store_i64(o, i, int_binary(op, load_i64(a, i), load_i64(b, i)));
    } else {
        /* f64 outputs keep the double result; narrower floats round it once more on store */
        #pragma omp parallel for
        for (size_t i = 0; i < o->size; i++)
            store_f64(o, i, float_binary(op, load_f64(a, i), load_f64(b, i)));
    }
}

ORC_API void orc_add(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_ADD, a, b, o); }
ORC_API void orc_sub(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_SUB, a, b, o); }
ORC_API void orc_mul(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_MUL, a, b, o); }
ORC_API void orc_div(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_DIV, a, b, o); }
/* Max / Min follow the same output-dtype dispatch (tensor_ops.c:1367-1403). */
ORC_API void orc_max(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_MAX, a, b, o); }
ORC_API void orc_min(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) { binary_forward(OP_MIN, a, b, o); }
/* Pow has no integer branch: always pow() in double and the generic store (tensor_ops.c:1355-1364). */
ORC_API void orc_pow(const OrcTensor* a, const OrcTensor* b, OrcTensor* o) {
    if (!a || !b || !o) return;
    #pragma omp parallel for
    for (size_t i = 0; i < o->size; i++) store_f64(o, i, pow(load_f64(a, i), load_f64(b, i)));
}

/* ------------------------------------------------------------------------------------------
 * The one-line unary operators (tensor_ops.c:595-604 is the shared shape: read as double, one
 * libm expression, generic store).  `which` selects the expression; the comments give the lines
 * of the reference's definitions.
 * ---------------------------------------------------------------------------------------- */
enum { UM_EXP, UM_LOG, UM_SQRT, UM_SIGMOID, UM_TANH, UM_NEG, UM_RECIPROCAL, UM_CEIL, UM_FLOOR, UM_SIN, UM_TAN, UM_ATAN,
       UM_SOFTPLUS, UM_SOFTSIGN, UM_HARD_SWISH, UM_ACOS, UM_ASIN, UM_COSH, UM_SINH, UM_ASINH, UM_ACOSH, UM_ATANH, UM_ROUND,
       UM_ERF, UM_GELU, UM_COUNT };

static double unary_math_value(int which, double v) {
    switch (which) {
        case UM_EXP:        return exp(v);                                   /* :1273 */
        case UM_LOG:        return log(v);                                   /* :1277 */
        case UM_SQRT:       return sqrt(v);                                  /* :1280 */
        case UM_SIGMOID:    return 1.0 / (1.0 + exp(-v));                    /* :1283 */
        case UM_TANH:       return tanh(v);                                  /* :1286 */
        case UM_NEG:        return -v;                                       /* :1484 */
        case UM_RECIPROCAL: return 1.0 / v;                                  /* :1487 */
        case UM_CEIL:       return ceil(v);                                  /* :1490 */
        case UM_FLOOR:      return floor(v);                                 /* :1493 */
        case UM_SIN:        return sin(v);                                   /* :1758 */
        case UM_TAN:        return tan(v);                                   /* :1759 */
        case UM_ATAN:       return atan(v);                                  /* :1760 */
        case UM_SOFTPLUS:   return log(1.0 + exp(v));                        /* :2622 */
        case UM_SOFTSIGN:   return v / (1.0 + fabs(v));                      /* :2625 */
        case UM_HARD_SWISH: return v * fmax(0.0, fmin(1.0, v / 6.0 + 0.5));  /* :2629 */
        case UM_ACOS:       return acos(v);                                  /* :2647 */
        case UM_ASIN:       return asin(v);                                  /* :2650 */
        case UM_COSH:       return cosh(v);                                  /* :2653 */
        case UM_SINH:       return sinh(v);                                  /* :2656 */
        case UM_ASINH:      return asinh(v);                                 /* :2659 */
        case UM_ACOSH:      return acosh(v);                                 /* :2662 */
        case UM_ATANH:      return atanh(v);                                 /* :2665 */
        case UM_ROUND:      return rint(v);                                  /* :3032 */
        case UM_ERF:        return erf(v);                                   /* :3035 */
        case UM_GELU:       return 0.5 * v * (1.0 + erf(v * 0.70710678118654752440));   /* :3340 */
        default:            return v;
    }
}

ORC_API void orc_unary_math(int which, const OrcTensor* x, OrcTensor* y) {
    if (!unary_args_ok(x, y) || which < 0 || which >= UM_COUNT) return;
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) store_f64(y, i, unary_math_value(which, load_f64(x, i)));
}

/* ------------------------------------------------------------------------------------------
 * QuantizeLinear / DequantizeLinear.  tensor_ops.c:999-1034.  X, scale and zero point are all
 * read at the same flat index (the caller pre-broadcasts them).
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_quantize_linear(const OrcTensor* x, const OrcTensor* s, const OrcTensor* z, OrcTensor* y) {
    if (!x || !s || !z || !y) return;
    #pragma omp parallel for
    for (size_t i = 0; i < y->size; i++) {
        const double sv = load_f64(s, i), zv = load_f64(z, i);
        double r = zv;
        if (sv != 0.0) r = rint(load_f64(x, i) / sv) + zv;
        store_f64(y, i, r);       /* fp8 targets therefore see an integer-valued input */
    }
}

ORC_API void orc_dequantize_linear(const OrcTensor* x, const OrcTensor* s, const OrcTensor* z, OrcTensor* y) {
    if (!x || !s || !z || !y) return;
    #pragma omp parallel for
    for (size_t i = 0; i < y->size; i++)
        store_f64(y, i, (load_f64(x, i) - load_f64(z, i)) * load_f64(s, i));
}

/* ------------------------------------------------------------------------------------------
 * Conv2d.  tensor_ops.c:1036-1114 (+ 687-700 for the zero-padded read).  NCHW, weights
 * [M, C/g, KH, KW]; reduction order ic -> kh -> kw in double; bias added after the reduction;
 * only pads[0] (top) and pads[1] (left) are read.
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_conv2d(const OrcTensor* x, const OrcTensor* w, const OrcTensor* b, OrcTensor* y,
                        const OrcConvParams* p) {
    const int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    const int M = w->shape[0], KH = w->shape[2], KW = w->shape[3];
    const int OH = y->shape[2], OW = y->shape[3];
    const int pt = p->pads[0], pl = p->pads[1];
    const int sh = p->strides[0], sw = p->strides[1];
    const int dh = p->dilations[0], dw = p->dilations[1];
    const int G = p->group, Cg = C / G, Mg = M / G;
    const int has_bias = b && b->data;

    #pragma omp parallel for collapse(2)
    for (int n = 0; n < N; n++)
    for (int m = 0; m < M; m++) {
        const int c0 = (m / Mg) * Cg;
        const double bias = has_bias ? load_f64(b, (size_t)m) : 0.0;
        for (int oh = 0; oh < OH; oh++)
        for (int ow = 0; ow < OW; ow++) {
            double acc = 0.0;
            for (int c = 0; c < Cg; c++)
            for (int kh = 0; kh < KH; kh++)
            for (int kw = 0; kw < KW; kw++) {
                const int ih = oh * sh + kh * dh - pt;
                const int iw = ow * sw + kw * dw - pl;
                double xv = 0.0;
                if (ih >= 0 && ih < H && iw >= 0 && iw < W)
                    xv = load_f64(x, (((size_t)n * C + (size_t)(c0 + c)) * H + (size_t)ih) * W + (size_t)iw);
                const double wv = load_f64(w, (((size_t)m * Cg + (size_t)c) * KH + (size_t)kh) * KW + (size_t)kw);
                acc += xv * wv;
            }
            store_f64(y, (((size_t)n * M + (size_t)m) * OH + (size_t)oh) * OW + (size_t)ow, acc + bias);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * MaxPool.  tensor_ops.c:1116-1165.  Scan kh -> kw from -Inf with a strict '>', skipping taps
 * outside the plane: NaN is never selected and an empty window yields -Inf.
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_max_pool(const OrcTensor* x, OrcTensor* y, const OrcPoolParams* p) {
    const int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    const int OH = y->shape[2], OW = y->shape[3];
    const int KH = p->kernel_shape[0], KW = p->kernel_shape[1];
    const int pt = p->pads[0], pl = p->pads[1];
    const int sh = p->strides[0], sw = p->strides[1];
    const int dh = p->dilations[0], dw = p->dilations[1];

    #pragma omp parallel for collapse(2)
    for (int n = 0; n < N; n++)
    for (int c = 0; c < C; c++) {
        const size_t in_plane = ((size_t)n * C + (size_t)c) * H * W;
        const size_t out_plane = ((size_t)n * C + (size_t)c) * OH * OW;
        for (int oh = 0; oh < OH; oh++)
        for (int ow = 0; ow < OW; ow++) {
            double best = -INFINITY;
            for (int kh = 0; kh < KH; kh++)
            for (int kw = 0; kw < KW; kw++) {
                const int ih = oh * sh + kh * dh - pt;
                const int iw = ow * sw + kw * dw - pl;
                if (ih < 0 || ih >= H || iw < 0 || iw >= W) continue;
                const double v = load_f64(x, in_plane + (size_t)ih * W + (size_t)iw);
                if (v > best) best = v;
            }
            store_f64(y, out_plane + (size_t)oh * OW + (size_t)ow, best);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Gemm.  tensor_ops.c:1167-1228.  Y = alpha * A' B' + beta * C with a sequential double
 * reduction over k, alpha*sum and beta*c rounded separately, C broadcast by shape.
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_gemm(const OrcTensor* a, const OrcTensor* b, const OrcTensor* c, OrcTensor* y,
                      float alpha, float beta, int transA, int transB) {
    const int M = transA ? a->shape[1] : a->shape[0];
    const int K = transA ? a->shape[0] : a->shape[1];
    const int N = transB ? b->shape[0] : b->shape[1];
    const size_t lda = (size_t)a->shape[1], ldb = (size_t)b->shape[1];
    const int has_c = c && c->data;

    #pragma omp parallel for collapse(2)
    for (int m = 0; m < M; m++)
    for (int n = 0; n < N; n++) {
        double acc = 0.0;
        for (int k = 0; k < K; k++) {
            const size_t ia = transA ? (size_t)k * lda + (size_t)m : (size_t)m * lda + (size_t)k;
            const size_t ib = transB ? (size_t)n * ldb + (size_t)k : (size_t)k * ldb + (size_t)n;
            acc += load_f64(a, ia) * load_f64(b, ib);
        }
        double r = (double)alpha * acc;
        if (has_c) {
            double cv = 0.0;
            if (c->size == 1) {
                cv = load_f64(c, 0);
            } else if (c->ndim == 1) {
                if (c->shape[0] == N)      cv = load_f64(c, (size_t)n);
                else if (c->shape[0] == M) cv = load_f64(c, (size_t)m);
            } else if (c->ndim >= 2) {
                const int R = c->shape[c->ndim - 2], Q = c->shape[c->ndim - 1];
                const int ir = (R == 1) ? 0 : m, iq = (Q == 1) ? 0 : n;
                /* the reference forms this index in int arithmetic */
                if (ir < R && iq < Q) cv = load_f64(c, (size_t)(ir * Q + iq));
            }
            r += (double)beta * cv;
        }
        store_f64(y, (size_t)m * N + (size_t)n, r);
    }
}

/* ------------------------------------------------------------------------------------------
 * Softmax.  tensor_ops.c:1231-1270.  View as [outer, inner, rem]; per (outer, rem): running
 * max from -DBL_MAX, then the sum of exp(v - max) in index order, then exp(v - max) / sum.
 * ---------------------------------------------------------------------------------------- */
ORC_API void orc_softmax(const OrcTensor* x, OrcTensor* y, int axis) {
    if (axis < 0) axis += x->ndim;
    const int inner = x->shape[axis];
    int outer = 1, rem = 1;
    for (int d = 0; d < axis; d++) outer *= x->shape[d];
    for (int d = axis + 1; d < x->ndim; d++) rem *= x->shape[d];

    #pragma omp parallel for collapse(2)
    for (int o = 0; o < outer; o++)
    for (int r = 0; r < rem; r++) {
        const size_t base = (size_t)o * inner * rem + (size_t)r;
        double top = -DBL_MAX;
        for (int j = 0; j < inner; j++) {
            const double v = load_f64(x, base + (size_t)j * rem);
            if (v > top) top = v;
        }
        double total = 0.0;
        for (int j = 0; j < inner; j++) total += exp(load_f64(x, base + (size_t)j * rem) - top);
        for (int j = 0; j < inner; j++) {
            const size_t idx = base + (size_t)j * rem;
            store_f64(y, idx, exp(load_f64(x, idx) - top) / total);
        }
    }
}

/* ------------------------------------------------------------------------------------------
 * Operators that surround the hot path in exported CNNs.
 * ---------------------------------------------------------------------------------------- */

/* Cast.  tensor_ops.c:1497-1519: float32 / float64 / float16 / bfloat16 sources going to an integer
   type are TRUNCATED toward zero (C cast to int64, then the saturating integer store); every other
   pair goes through a double and the generic store (so fp8 -> int rounds to nearest-even, and
   int64 -> int64 passes through a double). */
ORC_API void orc_cast(const OrcTensor* x, OrcTensor* y) {
    if (!unary_args_ok(x, y)) return;
    const int truncating = (x->dtype == DT_F32 || x->dtype == DT_F64 || x->dtype == DT_F16 || x->dtype == DT_BF16) &&
                           is_integer_dtype(y->dtype);
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) {
        const double v = load_f64(x, i);
        if (truncating) store_i64(y, i, trunc_to_i64_x86(v));
        else store_f64(y, i, v);
    }
}

/* Clip.  tensor_ops.c:1523-1543: compare in double, lower bound first; a NaN value or a NaN bound
   leaves the value as it is.  Bounds are optional and indexed like the input. */
ORC_API void orc_clip(const OrcTensor* x, OrcTensor* y, const OrcTensor* lo, const OrcTensor* hi) {
    if (!x || !y) return;
    const int has_lo = lo && lo->data, has_hi = hi && hi->data;
    #pragma omp parallel for
    for (size_t i = 0; i < y->size; i++) {
        double v = load_f64(x, i);
        if (has_lo) { const double b = load_f64(lo, i); if (v < b) v = b; }
        if (has_hi) { const double b = load_f64(hi, i); if (v > b) v = b; }
        store_f64(y, i, v);
    }
}

/* AveragePool.  tensor_ops.c:2735-2789: double sum over the taps inside the plane in kh -> kw
   order, divided by their number (or by the number of all taps with count_include_pad); a window
   without taps gives 0. */
ORC_API void orc_average_pool(const OrcTensor* x, OrcTensor* y, const OrcPoolParams* p, int count_include_pad) {
    if (!x || !y || !p) return;
    const int N = x->shape[0], C = x->shape[1], H = x->shape[2], W = x->shape[3];
    const int OH = y->shape[2], OW = y->shape[3];
    const int KH = p->kernel_shape[0], KW = p->kernel_shape[1];
    const int pt = p->pads[0], pl = p->pads[1];
    const int sh = p->strides[0], sw = p->strides[1];
    const int dh = p->dilations[0], dw = p->dilations[1];
    #pragma omp parallel for collapse(2)
    for (int n = 0; n < N; n++)
    for (int c = 0; c < C; c++) {
        const size_t in_plane = ((size_t)n * C + (size_t)c) * H * W;
        const size_t out_plane = ((size_t)n * C + (size_t)c) * OH * OW;
        for (int oh = 0; oh < OH; oh++)
        for (int ow = 0; ow < OW; ow++) {
            double sum = 0.0;
            int count = 0;
            for (int kh = 0; kh < KH; kh++)
            for (int kw = 0; kw < KW; kw++) {
                const int ih = oh * sh + kh * dh - pt;
                const int iw = ow * sw + kw * dw - pl;
                if (ih < 0 || ih >= H || iw < 0 || iw >= W) { if (count_include_pad) count++; continue; }
                sum += load_f64(x, in_plane + (size_t)ih * W + (size_t)iw);
                count++;
            }
            store_f64(y, out_plane + (size_t)oh * OW + (size_t)ow, count > 0 ? sum / count : 0.0);
        }
    }
}

/* GlobalAveragePool.  tensor_ops.c:2844-2868: 4-D inputs only; sequential double sum of each
   H x W plane divided by H * W. */
ORC_API void orc_global_average_pool(const OrcTensor* x, OrcTensor* y) {
    if (!x || !y || x->ndim != 4) return;
    const int planes = x->shape[0] * x->shape[1], spatial = x->shape[2] * x->shape[3];
    #pragma omp parallel for
    for (int n = 0; n < planes; n++) {
        double sum = 0.0;
        for (int i = 0; i < spatial; i++) sum += load_f64(x, (size_t)n * spatial + i);
        store_f64(y, (size_t)n, sum / spatial);
    }
}

/* BatchNormalization (inference).  tensor_ops.c:3041-3083: per channel a = scale / sqrt(var + eps)
   (eps arrives as a float and is widened), k = bias - mean * a; then y = x * a + k with separate
   roundings of the product and the sum (no fused multiply-add in the reference's build). */
ORC_API void orc_batch_norm(const OrcTensor* x, const OrcTensor* scale, const OrcTensor* bias, const OrcTensor* mean,
                            const OrcTensor* var, OrcTensor* y, float epsilon) {
    if (!x || !scale || !bias || !mean || !var || !y) return;
    const int N = x->shape[0], C = x->shape[1];
    size_t spatial = 1;
    for (int d = 2; d < x->ndim; d++) spatial *= (size_t)x->shape[d];
    #pragma omp parallel for collapse(2)
    for (int n = 0; n < N; n++)
    for (int c = 0; c < C; c++) {
        const double inv_std = 1.0 / sqrt(load_f64(var, c) + (double)epsilon);
        const double a = load_f64(scale, c) * inv_std;
        const double k = load_f64(bias, c) - load_f64(mean, c) * a;
        const size_t base = ((size_t)n * C + (size_t)c) * spatial;
        for (size_t i = 0; i < spatial; i++) {
            store_f64(y, base + i, load_f64(x, base + i) * a + k);       /* two roundings: this file is built with -ffp-contract=off */
        }
    }
}

/* MatMul with numpy-style broadcasting of the leading (batch) dimensions.  tensor_ops.c:1546-1606: every output
   element Y[..., m, n] is the double sum over k, in increasing k, of A[..., m, k] * B[..., k, n]; a batch
   dimension of extent 1 in an operand is read at index 0, and an operand of lower rank is aligned to the right. */
static size_t matmul_batch_offset(const OrcTensor* t, const int* y_coords, int y_ndim) {
    const int lead = t->ndim - 2, shift = y_ndim - t->ndim;
    size_t offset = 0;
    for (int d = 0; d < lead; d++) {
        const int c = t->shape[d] == 1 ? 0 : y_coords[d + shift];
        offset = offset * (size_t)t->shape[d] + (size_t)c;
    }
    return offset * (size_t)t->shape[t->ndim - 2] * (size_t)t->shape[t->ndim - 1];
}

ORC_API void orc_matmul(const OrcTensor* a, const OrcTensor* b, OrcTensor* y) {
    if (!a || !b || !y || y->ndim < 2 || y->ndim > 16 || a->ndim < 2 || b->ndim < 2) return;
    const int M = a->shape[a->ndim - 2], K = a->shape[a->ndim - 1], N = b->shape[b->ndim - 1];
    const size_t per_batch = (size_t)M * (size_t)N;
    const size_t batches = per_batch ? y->size / per_batch : 0;
    #pragma omp parallel for
    for (size_t bi = 0; bi < batches; bi++) {
        int coords[16];
        size_t rest = bi;
        for (int d = y->ndim - 3; d >= 0; d--) { coords[d] = (int)(rest % (size_t)y->shape[d]); rest /= (size_t)y->shape[d]; }
        const size_t a0 = matmul_batch_offset(a, coords, y->ndim), b0 = matmul_batch_offset(b, coords, y->ndim);
        for (int m = 0; m < M; m++)
        for (int n = 0; n < N; n++) {
            double sum = 0.0;
            for (int k = 0; k < K; k++) sum += load_f64(a, a0 + (size_t)m * K + k) * load_f64(b, b0 + (size_t)k * N + n);
            store_f64(y, bi * per_batch + (size_t)m * N + n, sum);
        }
    }
}

/* DynamicQuantizeLinear.  tensor_ops.c:3760-3809: the range [min(x, 0), max(x, 0)] (NaNs never win a comparison) is
   mapped onto 0..255: scale = (max - min) / 255 as a double (1 if that is 0), zero point = round-half-away(-min / scale)
   clamped to 0..255 and narrowed like a C cast, y = clamp(rint(x / scale) + zp, 0, 255) through the ordinary store.
   The division uses the DOUBLE scale; y_scale receives it rounded to its own type. */
/* The range pass alone: range[0] = min, range[1] = max over the elements, started at +-DBL_MAX like the reference
   (so an empty or all-NaN tensor leaves them there).  Ranges of row blocks combine with min / max. */
ORC_API void orc_dynamic_quantize_range(const OrcTensor* x, double* range) {
    double lo = DBL_MAX, hi = -DBL_MAX;
    for (size_t i = 0; x && i < x->size; i++) {
        const double v = load_f64(x, i);
        if (v < lo) lo = v;
        if (v > hi) hi = v;
    }
    range[0] = lo;
    range[1] = hi;
}

/* Everything after the range pass. */
ORC_API void orc_dynamic_quantize_apply(const OrcTensor* x, const double* range, OrcTensor* y, OrcTensor* y_scale, OrcTensor* y_zp) {
    if (!x || !y || !y_scale || !y_zp) return;
    const double lo = fmin(range[0], 0.0), hi = fmax(range[1], 0.0);
    double scale = (hi - lo) / 255.0;
    if (scale == 0.0) scale = 1.0;
    double zd = round(0.0 - lo / scale);
    if (zd < 0.0) zd = 0.0;
    if (zd > 255.0) zd = 255.0;
    const uint8_t zp = (uint8_t)trunc_to_i64_x86(zd);          /* a NaN (infinite range) narrows to 0 */
    store_f64(y_scale, 0, scale);
    if (y_zp->dtype == DT_U8) ((uint8_t*)y_zp->data)[0] = zp;
    else store_f64(y_zp, 0, (double)zp);
    #pragma omp parallel for
    for (size_t i = 0; i < x->size; i++) {
        double q = rint(load_f64(x, i) / scale) + (double)zp;
        if (q < 0.0) q = 0.0;
        if (q > 255.0) q = 255.0;
        store_f64(y, i, q);
    }
}

ORC_API void orc_dynamic_quantize_linear(const OrcTensor* x, OrcTensor* y, OrcTensor* y_scale, OrcTensor* y_zp) {
    if (!x || !y || !y_scale || !y_zp) return;
    double range[2];
    orc_dynamic_quantize_range(x, range);
    orc_dynamic_quantize_apply(x, range, y, y_scale, y_zp);
}

/* Flatten / Reshape: a byte copy.  tensor_ops.c:1289-1299 */
ORC_API void orc_flatten(const OrcTensor* x, OrcTensor* y) {
    if (!x || !y || x->size != y->size) return;
    memcpy(y->data, x->data, x->size * orc_dtype_size(x->dtype));
}
