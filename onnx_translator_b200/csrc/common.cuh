// Shared declarations of the operator library: runtime context, error reporting, dtype traits,
// the device-side codecs, and the broadcast-operand descriptor used by every elementwise kernel.
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <stdint.h>
#include <stdio.h>

#include "tensor_ops_b200.h"

#define TOPS_API extern "C" __attribute__((visibility("default")))

namespace tops {

// ---------------------------------------------------------------------------------------------
// Runtime context (runtime.cu)
// ---------------------------------------------------------------------------------------------
constexpr int kMaxDevices = 16;
constexpr int kNumSMs = 148;            // B200: 2 dies x 74 SMs; grids are sized in multiples of it

struct DeviceState {
    bool         ready = false;
    cudaStream_t own_stream = nullptr;
    double*      cos_lut = nullptr;     // 4097 doubles, device memory
    int          sm_count = kNumSMs;
};

// Makes the calling thread's device current and returns its state (nullptr + error if no device).
DeviceState* acquire_device();
cudaStream_t current_stream();
bool         managed_mode();
void         finish_op();                 // managed mode: synchronise so the host may read results
void         set_error(int code, const char* fmt, ...);
bool         check_cuda(cudaError_t e, const char* what);
void         zero_fill(Tensor* t);        // best effort, used on rejected calls
const double* cos_lut_device();           // uploads on first use
int*         device_status_word();        // device pointer to the host-visible status word (may be null)
int*         device_status_word_if_created();   // as above, but never allocates (null until first created)
void         poll_device_status();        // host: turn a raised status word into an error
// Opt-in for more than 48 KB of dynamic shared memory.  The attribute belongs to the (kernel, device) pair, so
// it is recorded per device: the first launch of `kernel` on each device sets it, with that device current.
bool         ensure_dynamic_smem(const void* kernel, size_t bytes);

#define TOPS_CUDA_OK(expr) ::tops::check_cuda((expr), #expr)
#define TOPS_CHECK_LAUNCH(name) ::tops::check_cuda(cudaGetLastError(), name)

// ---------------------------------------------------------------------------------------------
// dtype traits
// ---------------------------------------------------------------------------------------------
__host__ __device__ constexpr int dtype_bytes(int dt) {
    return (dt == DTYPE_FLOAT16 || dt == DTYPE_BFLOAT16 || dt == DTYPE_INT16) ? 2
         : (dt == DTYPE_FLOAT32 || dt == DTYPE_INT32) ? 4
         : (dt == DTYPE_FLOAT64 || dt == DTYPE_INT64) ? 8
         : (dt >= 0 && dt <= DTYPE_INT64) ? 1 : 4;
}
__host__ __device__ constexpr bool dtype_is_int(int dt) { return dt >= DTYPE_INT4 && dt <= DTYPE_INT64; }
__host__ __device__ constexpr bool dtype_valid(int dt) { return dt >= 0 && dt <= DTYPE_INT64; }
// Every value of the type is exactly representable in float32.
__host__ __device__ constexpr bool dtype_exact_in_f32(int dt) {
    return dt != DTYPE_FLOAT64 && dt != DTYPE_INT32 && dt != DTYPE_INT64;
}
// Integer types whose values fit 16 bits (sums / products of two of them fit int32).
__host__ __device__ constexpr bool dtype_is_narrow_int(int dt) {
    return dt == DTYPE_INT4 || dt == DTYPE_INT8 || dt == DTYPE_UINT8 || dt == DTYPE_INT16;
}

// ---------------------------------------------------------------------------------------------
// Codecs.  The reference's encoders differ from IEEE / hardware converts in a few places
// (tensor_ops.c:104-152, 192-210, 258-287, 318-347):
//   fp16: |x| < 2^-24 -> +-0 (IEEE would round (2^-25, 2^-24) up); NaN -> sign|0x7FFF
//   bf16: NaN -> (bits>>16)|0x40
//   e4m3: |x| < 2^-6 -> +-0 (no subnormal outputs); overflow/Inf saturate to 0x7E; NaN -> 0x7F|sign
//   e5m2: |x| < 2^-14 -> +-0; overflow -> Inf 0x7C (no saturation); NaN -> 0x7D|sign
// The fast encoders below use the hardware converts plus these fix-ups; the bit-level
// restatements (encode_*_bits) exist so the two can be compared exhaustively on the device.
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t f32_bits(float f) { return __float_as_uint(f); }

__device__ __forceinline__ uint16_t encode_f16(float f) {
    const uint32_t u = f32_bits(f);
    const uint32_t mag = u & 0x7FFFFFFFu;
    const uint16_t sign = (uint16_t)((u >> 16) & 0x8000u);
    if (mag > 0x7F800000u) return sign | 0x7FFFu;
    if (mag < 0x33800000u) return sign;                       // below 2^-24
    return __half_as_ushort(__float2half_rn(f));
}
__device__ __forceinline__ float decode_f16(uint16_t h) { return __half2float(__ushort_as_half(h)); }

__device__ __forceinline__ uint16_t encode_bf16(float f) {
    const uint32_t u = f32_bits(f);
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)((u >> 16) | 0x0040u);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}
__device__ __forceinline__ float decode_bf16(uint16_t b) { return __uint_as_float((uint32_t)b << 16); }

__device__ __forceinline__ uint8_t encode_e4m3(float f) {
    const uint32_t u = f32_bits(f);
    const uint32_t mag = u & 0x7FFFFFFFu;
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    if (mag > 0x7F800000u) return sign | 0x7Fu;
    if (mag < 0x3C800000u) return sign;                       // below 2^-6
    return (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ float decode_e4m3(uint8_t c) {
    return __half2float(__half(__nv_cvt_fp8_to_halfraw(c, __NV_E4M3)));
}

__device__ __forceinline__ uint8_t encode_e5m2(float f) {
    const uint32_t u = f32_bits(f);
    const uint32_t mag = u & 0x7FFFFFFFu;
    const uint8_t sign = (uint8_t)((u >> 24) & 0x80u);
    if (mag > 0x7F800000u) return sign | 0x7Du;
    if (mag < 0x38800000u) return sign;                       // below 2^-14
    if (mag >= 0x47700000u) return sign | 0x7Cu;              // >= 61440 rounds past the largest finite
    return (uint8_t)__nv_cvt_float_to_fp8(f, __NV_SATFINITE, __NV_E5M2);
}
__device__ __forceinline__ float decode_e5m2(uint8_t c) {      // e5m2 is the top byte of fp16
    return __half2float(__ushort_as_half((uint16_t)c << 8));
}

// Bit-level restatement of the reference's small-float encoders (one parametric routine).
template <int EBITS, int MBITS, int BIAS, int FLUSH_EXP, bool IEEE_SPECIALS, bool SATURATE, uint32_t NAN_CODE>
__device__ __forceinline__ uint32_t encode_small_bits(float f) {
    const uint32_t u = f32_bits(f);
    constexpr int total = 1 + EBITS + MBITS;
    const uint32_t sign = (u >> 31) << (total - 1);
    const uint32_t e32 = (u >> 23) & 0xFFu, m32 = u & 0x7FFFFFu;
    constexpr uint32_t emax = (1u << EBITS) - 1u;
    constexpr uint32_t inf_code = emax << MBITS;
    constexpr uint32_t max_finite = IEEE_SPECIALS ? inf_code - 1u : (inf_code | ((1u << MBITS) - 2u));
    constexpr uint32_t over = SATURATE ? max_finite : inf_code;
    if (e32 == 255u) return m32 ? (sign | NAN_CODE) : (sign | over);
    if (e32 == 0u) return sign;
    const int unbiased = (int)e32 - 127;
    if (unbiased < FLUSH_EXP) return sign;
    int te = unbiased + BIAS, drop = 23 - MBITS;
    if (te <= 0) { drop += 1 - te; te = 0; }
    const uint32_t sig = m32 | 0x800000u;
    uint32_t kept = sig >> drop;
    const uint32_t rem = sig & ((1u << drop) - 1u), half = 1u << (drop - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    const uint32_t code = (te == 0) ? kept : (((uint32_t)(te - 1) << MBITS) + kept);
    return code > max_finite ? (sign | over) : (sign | code);
}
__device__ __forceinline__ uint32_t encode_f16_bits(float f)  { return encode_small_bits<5, 10, 15, -24, true, false, 0x7FFFu>(f); }
__device__ __forceinline__ uint32_t encode_e4m3_bits(float f) { return encode_small_bits<4, 3, 7, -6, false, true, 0x7Fu>(f); }
__device__ __forceinline__ uint32_t encode_e5m2_bits(float f) { return encode_small_bits<5, 2, 15, -14, true, false, 0x7Du>(f); }

// (int64_t)x as an x86-64 build performs it: NaN, +-Inf and out-of-range give INT64_MIN
// ("integer indefinite"), everything else truncates.  Inputs here are already integral.
__device__ __forceinline__ long long x86_f64_to_i64(double v) {
    if (!(v >= -9223372036854775808.0 && v < 9223372036854775808.0)) return (long long)0x8000000000000000ull;
    return __double2ll_rz(v);
}
__device__ __forceinline__ long long x86_f32_to_i64(float v) {
    if (!(v >= -9223372036854775808.0f && v < 9223372036854775808.0f)) return (long long)0x8000000000000000ull;
    return __float2ll_rz(v);
}

__device__ __forceinline__ int int4_value(int raw) {
    const int v = raw & 0x0F;
    return (v & 0x08) ? v - 16 : v;
}

// Storage type per dtype code.
template <int DT> struct Storage { using type = uint8_t; };
template <> struct Storage<DTYPE_FLOAT16>  { using type = uint16_t; };
template <> struct Storage<DTYPE_BFLOAT16> { using type = uint16_t; };
template <> struct Storage<DTYPE_INT16>    { using type = int16_t; };
template <> struct Storage<DTYPE_FLOAT32>  { using type = float; };
template <> struct Storage<DTYPE_INT32>    { using type = int32_t; };
template <> struct Storage<DTYPE_FLOAT64>  { using type = double; };
template <> struct Storage<DTYPE_INT64>    { using type = long long; };
template <> struct Storage<DTYPE_INT8>     { using type = int8_t; };
template <> struct Storage<DTYPE_INT4>     { using type = int8_t; };

// Decode one stored element to float / double / int64 (tensor_ops.c:488-546).
template <int DT> __device__ __forceinline__ float to_f32(typename Storage<DT>::type s) {
    if constexpr (DT == DTYPE_FLOAT8_E4M3) return decode_e4m3(s);
    else if constexpr (DT == DTYPE_FLOAT8_E5M2) return decode_e5m2(s);
    else if constexpr (DT == DTYPE_FLOAT16) return decode_f16(s);
    else if constexpr (DT == DTYPE_BFLOAT16) return decode_bf16(s);
    else if constexpr (DT == DTYPE_INT4) return (float)int4_value(s);
    else return (float)s;
}
template <int DT> __device__ __forceinline__ double to_f64(typename Storage<DT>::type s) {
    if constexpr (DT == DTYPE_FLOAT64) return s;
    else if constexpr (DT == DTYPE_INT32 || DT == DTYPE_INT64) return (double)s;
    else return (double)to_f32<DT>(s);
}
template <int DT> __device__ __forceinline__ long long to_i64(typename Storage<DT>::type s) {
    if constexpr (DT == DTYPE_INT4) return int4_value(s);
    else if constexpr (dtype_is_int(DT)) return (long long)s;
    else if constexpr (DT == DTYPE_FLOAT64) return x86_f64_to_i64(rint(s));
    else return x86_f32_to_i64(rintf(to_f32<DT>(s)));
}
template <int DT> __device__ __forceinline__ int to_i32_narrow(typename Storage<DT>::type s) {
    if constexpr (DT == DTYPE_INT4) return int4_value(s);
    else return (int)s;
}

__device__ __forceinline__ long long clamp_ll(long long v, long long lo, long long hi) {
    return v < lo ? lo : (v > hi ? hi : v);
}

// Encode to storage (tensor_ops.c:552-588).
template <int DT> __device__ __forceinline__ typename Storage<DT>::type from_i64(long long v) {
    if constexpr (DT == DTYPE_INT4) return (int8_t)clamp_ll(v, -8, 7);
    else if constexpr (DT == DTYPE_INT8) return (int8_t)clamp_ll(v, -128, 127);
    else if constexpr (DT == DTYPE_UINT8) return (uint8_t)clamp_ll(v, 0, 255);
    else if constexpr (DT == DTYPE_INT16) return (int16_t)clamp_ll(v, -32768, 32767);
    else if constexpr (DT == DTYPE_INT32) return (int32_t)clamp_ll(v, -2147483648ll, 2147483647ll);
    else if constexpr (DT == DTYPE_INT64) return v;
    else if constexpr (DT == DTYPE_FLOAT64) return (double)v;
    else if constexpr (DT == DTYPE_FLOAT32) return (float)v;
    else if constexpr (DT == DTYPE_FLOAT16) return encode_f16((float)v);
    else if constexpr (DT == DTYPE_BFLOAT16) return encode_bf16((float)v);
    else if constexpr (DT == DTYPE_FLOAT8_E4M3) return encode_e4m3((float)v);
    else return encode_e5m2((float)v);
}
template <int DT> __device__ __forceinline__ typename Storage<DT>::type from_i32(int v) {
    if constexpr (DT == DTYPE_INT4) return (int8_t)min(max(v, -8), 7);
    else if constexpr (DT == DTYPE_INT8) return (int8_t)min(max(v, -128), 127);
    else if constexpr (DT == DTYPE_UINT8) return (uint8_t)min(max(v, 0), 255);
    else if constexpr (DT == DTYPE_INT16) return (int16_t)min(max(v, -32768), 32767);
    else return from_i64<DT>((long long)v);
}
template <int DT> __device__ __forceinline__ typename Storage<DT>::type from_f32(float v) {
    if constexpr (DT == DTYPE_FLOAT32) return v;
    else if constexpr (DT == DTYPE_FLOAT64) return (double)v;
    else if constexpr (DT == DTYPE_FLOAT16) return encode_f16(v);
    else if constexpr (DT == DTYPE_BFLOAT16) return encode_bf16(v);
    else if constexpr (DT == DTYPE_FLOAT8_E4M3) return encode_e4m3(v);
    else if constexpr (DT == DTYPE_FLOAT8_E5M2) return encode_e5m2(v);
    else return from_i64<DT>(x86_f64_to_i64(rint((double)v)));
}
template <int DT> __device__ __forceinline__ typename Storage<DT>::type from_f64(double v) {
    if constexpr (DT == DTYPE_FLOAT64) return v;
    else if constexpr (dtype_is_int(DT)) return from_i64<DT>(x86_f64_to_i64(rint(v)));
    else return from_f32<DT>(__double2float_rn(v));
}

// Runtime-dtype element access for the generic (any dtype combination) kernels.
__device__ __forceinline__ double load_f64_rt(const void* p, int dt, size_t i) {
    switch (dt) {
        case DTYPE_FLOAT8_E4M3: return (double)decode_e4m3(((const uint8_t*)p)[i]);
        case DTYPE_FLOAT8_E5M2: return (double)decode_e5m2(((const uint8_t*)p)[i]);
        case DTYPE_FLOAT16:     return (double)decode_f16(((const uint16_t*)p)[i]);
        case DTYPE_BFLOAT16:    return (double)decode_bf16(((const uint16_t*)p)[i]);
        case DTYPE_FLOAT32:     return (double)((const float*)p)[i];
        case DTYPE_FLOAT64:     return ((const double*)p)[i];
        case DTYPE_INT4:        return (double)int4_value(((const int8_t*)p)[i]);
        case DTYPE_INT8:        return (double)((const int8_t*)p)[i];
        case DTYPE_UINT8:       return (double)((const uint8_t*)p)[i];
        case DTYPE_INT16:       return (double)((const int16_t*)p)[i];
        case DTYPE_INT32:       return (double)((const int32_t*)p)[i];
        case DTYPE_INT64:       return (double)((const long long*)p)[i];
        default:                return 0.0;
    }
}
__device__ __forceinline__ long long load_i64_rt(const void* p, int dt, size_t i) {
    switch (dt) {
        case DTYPE_FLOAT8_E4M3: return x86_f32_to_i64(rintf(decode_e4m3(((const uint8_t*)p)[i])));
        case DTYPE_FLOAT8_E5M2: return x86_f32_to_i64(rintf(decode_e5m2(((const uint8_t*)p)[i])));
        case DTYPE_FLOAT16:     return x86_f32_to_i64(rintf(decode_f16(((const uint16_t*)p)[i])));
        case DTYPE_BFLOAT16:    return x86_f32_to_i64(rintf(decode_bf16(((const uint16_t*)p)[i])));
        case DTYPE_FLOAT32:     return x86_f32_to_i64(rintf(((const float*)p)[i]));
        case DTYPE_FLOAT64:     return x86_f64_to_i64(rint(((const double*)p)[i]));
        case DTYPE_INT4:        return int4_value(((const int8_t*)p)[i]);
        case DTYPE_INT8:        return ((const int8_t*)p)[i];
        case DTYPE_UINT8:       return ((const uint8_t*)p)[i];
        case DTYPE_INT16:       return ((const int16_t*)p)[i];
        case DTYPE_INT32:       return ((const int32_t*)p)[i];
        case DTYPE_INT64:       return ((const long long*)p)[i];
        default:                return 0;
    }
}
__device__ __forceinline__ void store_i64_rt(void* p, int dt, size_t i, long long v) {
    switch (dt) {
        case DTYPE_FLOAT8_E4M3: ((uint8_t*)p)[i] = from_i64<DTYPE_FLOAT8_E4M3>(v); break;
        case DTYPE_FLOAT8_E5M2: ((uint8_t*)p)[i] = from_i64<DTYPE_FLOAT8_E5M2>(v); break;
        case DTYPE_FLOAT16:     ((uint16_t*)p)[i] = from_i64<DTYPE_FLOAT16>(v); break;
        case DTYPE_BFLOAT16:    ((uint16_t*)p)[i] = from_i64<DTYPE_BFLOAT16>(v); break;
        case DTYPE_FLOAT32:     ((float*)p)[i] = (float)v; break;
        case DTYPE_FLOAT64:     ((double*)p)[i] = (double)v; break;
        case DTYPE_INT4:        ((int8_t*)p)[i] = from_i64<DTYPE_INT4>(v); break;
        case DTYPE_INT8:        ((int8_t*)p)[i] = from_i64<DTYPE_INT8>(v); break;
        case DTYPE_UINT8:       ((uint8_t*)p)[i] = from_i64<DTYPE_UINT8>(v); break;
        case DTYPE_INT16:       ((int16_t*)p)[i] = from_i64<DTYPE_INT16>(v); break;
        case DTYPE_INT32:       ((int32_t*)p)[i] = from_i64<DTYPE_INT32>(v); break;
        case DTYPE_INT64:       ((long long*)p)[i] = v; break;
        default: break;
    }
}
__device__ __forceinline__ void store_f64_rt(void* p, int dt, size_t i, double v) {
    switch (dt) {
        case DTYPE_FLOAT8_E4M3: ((uint8_t*)p)[i] = from_f64<DTYPE_FLOAT8_E4M3>(v); break;
        case DTYPE_FLOAT8_E5M2: ((uint8_t*)p)[i] = from_f64<DTYPE_FLOAT8_E5M2>(v); break;
        case DTYPE_FLOAT16:     ((uint16_t*)p)[i] = from_f64<DTYPE_FLOAT16>(v); break;
        case DTYPE_BFLOAT16:    ((uint16_t*)p)[i] = from_f64<DTYPE_BFLOAT16>(v); break;
        case DTYPE_FLOAT32:     ((float*)p)[i] = __double2float_rn(v); break;
        case DTYPE_FLOAT64:     ((double*)p)[i] = v; break;
        default:                if (dtype_is_int(dt)) store_i64_rt(p, dt, i, x86_f64_to_i64(rint(v))); break;
    }
}

// ---------------------------------------------------------------------------------------------
// Broadcast operands.  An operand is described against the flat index space of the output:
// either FLAT (same element count: element i of the output pairs with element i of the operand)
// or by collapsed dimensions with per-dimension strides (0 where the operand is broadcast).
// All indices are 32-bit: the host splits launches so that one launch covers < 2^31 elements.
// ---------------------------------------------------------------------------------------------
constexpr int kMaxCollapsedDims = 16;   // the reference's MAX_NDIM: an alternating broadcast cannot collapse

struct FastDiv {            // n / d for n < 2^31 via multiply-high
    uint32_t d = 1, mul = 0, shift = 0;
    __host__ void set(uint32_t divisor) {
        d = divisor; mul = 0; shift = 0;
        if (d <= 1) { d = 1; return; }
        uint32_t s = 0;                       // smallest s with 2^s >= d
        while ((1ull << s) < d) s++;
        shift = s;
        mul = (uint32_t)(((1ull << (31 + s)) + d - 1) / d);   // ceil(2^(31+s) / d) < 2^32
    }
    __device__ __forceinline__ uint32_t div(uint32_t n) const {
        return d == 1 ? n : (uint32_t)(__umulhi(n, mul) >> (shift - 1));
    }
};

struct Operand {
    const void* ptr = nullptr;
    int flat = 1;                           // 1: index == output index
    int nd = 0;                             // collapsed dims (outermost first) when !flat
    int stride[kMaxCollapsedDims] = {0};    // element strides of THIS operand per collapsed dim
};

struct Geometry {                           // collapsed output shape shared by all operands
    int nd = 1;
    uint32_t size[kMaxCollapsedDims] = {1};
    FastDiv div[kMaxCollapsedDims];
};

// Offset of output element `i` inside a broadcast operand, plus the coordinate in the innermost
// collapsed dimension (so the caller can tell whether a run of elements stays inside it).
__device__ __forceinline__ uint32_t operand_offset(const Geometry& g, const Operand& op, uint32_t i, uint32_t& inner_pos) {
    uint32_t off = 0, rest = i;
    for (int d = g.nd - 1; d > 0; --d) {
        const uint32_t q = g.div[d].div(rest);
        const uint32_t r = rest - q * g.size[d];
        if (d == g.nd - 1) inner_pos = r;
        off += r * (uint32_t)op.stride[d];
        rest = q;
    }
    if (g.nd == 1) inner_pos = rest;
    off += rest * (uint32_t)op.stride[0];
    return off;
}

// Host side (broadcast.cu)
struct ShapeView { const int* shape; int ndim; size_t size; };
// Builds the shared geometry and one Operand per input for an output of shape `out`.
// Returns false when an input cannot be broadcast to the output shape.
bool plan_broadcast(const ShapeView& out, const ShapeView* ins, int n_in, Geometry* geom, Operand* ops);

inline int grid_for(size_t work_items, int threads, int sm_count, int ctas_per_sm) {
    size_t blocks = (work_items + (size_t)threads - 1) / (size_t)threads;
    size_t cap = (size_t)sm_count * (size_t)ctas_per_sm;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    return (int)blocks;
}

}  // namespace tops
