// QuantizeLinear / DequantizeLinear (tensor_ops.c:999-1034) for the two shapes of scale that dominate real graphs,
// written as loops a thread stays in: float32 values against 8-bit codes with
//   * one scale and one zero point for the whole tensor, or
//   * one per element of the innermost dimension (per-axis on the last axis).
// Everything that does not depend on the element -- reciprocal of the scale, zero point folded into the rounding
// constant -- is computed once per thread instead of once per run, and a thread moves 16 elements per step
// (64 bytes of float32, 16 bytes of codes).  The arithmetic is that of the general bodies (qdq_math.cuh): rounding by
// adding 1.5 * 2^23, a tie margin test, the reference's double division for the rare undecided run.
// For the per-axis form the grid is sized so that a thread meets the same 16 columns on every step.
#include "elementwise.cuh"
#include "qdq_math.cuh"

namespace tops {

template <int DT> __device__ __forceinline__ float zero_point_value(const void* p, size_t i) {
    if constexpr (DT == DTYPE_INT8) return (float)((const int8_t*)p)[i];
    else if constexpr (DT == DTYPE_UINT8) return (float)((const uint8_t*)p)[i];
    else return to_f32<DT>(((const typename Storage<DT>::type*)p)[i]);
}

// The reference's double division for one element, out of line: it runs for about one run in a thousand.
template <int DO>
static __device__ __noinline__ uint32_t quantize_exact_code(float x, float s, float z) {
    const typename Storage<DO>::type code = quantize_exact<DO>((double)x, (double)s, (double)z);
    return (uint32_t)*reinterpret_cast<const uint8_t*>(&code);
}

// What a kernel keeps per zero point: for float8 codes the value itself; for integer codes the bit pattern of
// (zero point - bits of 1.5 * 2^23), which added to the bits of the rounding sum gives the code before saturation.
template <int DO, int DZ> __device__ __forceinline__ float zero_point_term(const void* p, size_t i) {
    const float z = zero_point_value<DZ>(p, i);
    if constexpr (DO == DTYPE_INT8 || DO == DTYPE_UINT8) return __int_as_float((int)z - 0x4B400000);
    else return z;
}

// 16 values -> 16 codes.  `inv`, `zf` (zero_point_term): per element when PER_COLUMN, else entry 0 serves all.
template <int DO, bool PER_COLUMN>
__device__ __forceinline__ bool quantize16(const float (&x)[16], const float* inv, const float* zf, uint32_t (&words)[4]) {
    constexpr bool kFp8 = DO == DTYPE_FLOAT8_E4M3 || DO == DTYPE_FLOAT8_E5M2;
    bool all_ok = true;
    if constexpr (kFp8) {
        float fr[16];
        #pragma unroll
        for (int j = 0; j < 16; j++) {
            const float q = __fmul_rn(x[j], inv[PER_COLUMN ? j : 0]);
            const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
            all_ok = all_ok & (fmaf(fabsf(q), 1.9073486e-6f, fabsf(__fsub_rn(q, rq))) < 0.5f);
            if constexpr (DO == DTYPE_FLOAT8_E5M2) all_ok = all_ok & (fabsf(q) < 57000.0f);     // beyond: the reference overflows to infinity
            fr[j] = __fadd_rn(rq, zf[PER_COLUMN ? j : 0]);
        }
        #pragma unroll
        for (int j = 0; j < 16; j += 4) {
            const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(fr[j], fr[j + 1]), __NV_SATFINITE, DO == DTYPE_FLOAT8_E4M3 ? __NV_E4M3 : __NV_E5M2);
            const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(fr[j + 2], fr[j + 3]), __NV_SATFINITE, DO == DTYPE_FLOAT8_E4M3 ? __NV_E4M3 : __NV_E5M2);
            words[j >> 2] = lo | (hi << 16);
        }
    } else {
        int v[16];
        #pragma unroll
        for (int j = 0; j < 16; j++) {
            const float q = __fmul_rn(x[j], inv[PER_COLUMN ? j : 0]);
            const float t = __fadd_rn(q, 12582912.0f);
            const float d = __fsub_rn(q, __fsub_rn(t, 12582912.0f));
            all_ok = all_ok & (fmaf(fabsf(q), 1.9073486e-6f, fabsf(d)) < 0.5f);
            v[j] = __float_as_int(t) + __float_as_int(zf[PER_COLUMN ? j : 0]);
        }
        #pragma unroll
        for (int j = 0; j < 16; j += 4)
            words[j >> 2] = DO == DTYPE_INT8 ? pack_sat_s8x4(v[j], v[j + 1], v[j + 2], v[j + 3]) : pack_sat_u8x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    }
    return all_ok;
}

// One step of 16 elements at `first`; `col` is the first column's index into scale / zero (0 for the per-tensor form).
template <int DO, int DZ, bool PER_COLUMN>
__device__ __forceinline__ void quantize_step(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                              const void* __restrict__ zero, size_t first, size_t col, const float* inv, const float* zf) {
    float v[16];
    #pragma unroll
    for (int k = 0; k < 4; k++) {
        const float4 f = __ldcs(reinterpret_cast<const float4*>(x + first) + k);
        v[4 * k] = f.x; v[4 * k + 1] = f.y; v[4 * k + 2] = f.z; v[4 * k + 3] = f.w;
    }
    uint32_t words[4];
    if (!quantize16<DO, PER_COLUMN>(v, inv, zf, words)) {          // rare: some element sits on a rounding tie, is huge or not finite
        #pragma unroll
        for (int j = 0; j < 16; j++) {
            const size_t c = PER_COLUMN ? col + j : 0;
            const uint32_t code = quantize_exact_code<DO>(v[j], scale[c], zero_point_value<DZ>(zero, c));
            if ((j & 3) == 0) words[j >> 2] = code;
            else words[j >> 2] |= code << (8 * (j & 3));
        }
    }
    __stcs(reinterpret_cast<uint4*>(y + first), make_uint4(words[0], words[1], words[2], words[3]));
}

template <int DO, int DZ>
__global__ void __launch_bounds__(256) quantize_per_tensor_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                                                  const void* __restrict__ zero, size_t n) {
    wait_for_previous_kernel();
    float inv[1] = {quantize_reciprocal(__ldg(scale))};
    float zf[1] = {zero_point_term<DO, DZ>(zero, 0)};
    const size_t runs = n / 16, step = (size_t)gridDim.x * blockDim.x;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += step)
        quantize_step<DO, DZ, false>(x, y, scale, zero, r * 16, 0, inv, zf);
    if (blockIdx.x == 0 && threadIdx.x == 0)                             // the last, incomplete run
        for (size_t i = runs * 16; i < n; i++) {
            const typename Storage<DO>::type code = quantize_exact<DO>((double)x[i], (double)scale[0], (double)zero_point_value<DZ>(zero, 0));
            y[i] = *reinterpret_cast<const uint8_t*>(&code);
        }
}

// rows x cols, scale / zero of length cols; cols is a multiple of 16 and the thread count a multiple of cols / 16.
template <int DO, int DZ>
__global__ void __launch_bounds__(256) quantize_per_column_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                                                  const void* __restrict__ zero, size_t rows, uint32_t cols) {
    wait_for_previous_kernel();
    const uint32_t groups = cols / 16;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, threads = (size_t)gridDim.x * blockDim.x;
    const uint32_t col = (uint32_t)(tid % groups) * 16;
    float inv[16], zf[16];
    #pragma unroll
    for (int j = 0; j < 16; j++) { inv[j] = quantize_reciprocal(__ldg(scale + col + j)); zf[j] = zero_point_term<DO, DZ>(zero, col + j); }
    for (size_t row = tid / groups; row < rows; row += threads / groups)
        quantize_step<DO, DZ, true>(x, y, scale, zero, row * cols + col, col, inv, zf);
}

// ---- Dequantize: 16 codes -> 16 float32 -------------------------------------------------------------------------------
template <int DX, bool PER_COLUMN>
__device__ __forceinline__ void dequantize_step(const uint8_t* __restrict__ x, float* __restrict__ y, size_t first, const float* s, const float* zf) {
    const uint4 raw = __ldcs(reinterpret_cast<const uint4*>(x + first));
    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float f[16];
    #pragma unroll
    for (int k = 0; k < 4; k++) {
        if constexpr (DX == DTYPE_INT8 || DX == DTYPE_UINT8) {
            // the byte becomes the low mantissa byte of 2^23 (signed bytes biased by 128 first); the bias leaves with the zero point
            const uint32_t word = DX == DTYPE_INT8 ? (w[k] ^ 0x80808080u) : w[k];
            const float bias = DX == DTYPE_INT8 ? 8388736.0f : 8388608.0f;
            f[4 * k]     = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540)), bias);
            f[4 * k + 1] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7541)), bias);
            f[4 * k + 2] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7542)), bias);
            f[4 * k + 3] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7543)), bias);
        } else {
            #pragma unroll
            for (int h = 0; h < 2; h++) {                        // two float8 codes per hardware convert
                const uint16_t two = (uint16_t)(w[k] >> (16 * h));
                uint32_t half2_bits;
                if constexpr (DX == DTYPE_FLOAT8_E4M3) {
                    const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(two, __NV_E4M3);
                    half2_bits = (uint32_t)hr.x | ((uint32_t)hr.y << 16);
                } else {
                    half2_bits = __byte_perm((uint32_t)two, 0u, 0x1404);       // an e5m2 code is the upper byte of a float16
                }
                const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&half2_bits));
                f[4 * k + 2 * h] = p.x; f[4 * k + 2 * h + 1] = p.y;
            }
        }
    }
    #pragma unroll
    for (int k = 0; k < 4; k++) {
        float4 out;
        out.x = __fmul_rn(__fsub_rn(f[4 * k], zf[PER_COLUMN ? 4 * k : 0]), s[PER_COLUMN ? 4 * k : 0]);
        out.y = __fmul_rn(__fsub_rn(f[4 * k + 1], zf[PER_COLUMN ? 4 * k + 1 : 0]), s[PER_COLUMN ? 4 * k + 1 : 0]);
        out.z = __fmul_rn(__fsub_rn(f[4 * k + 2], zf[PER_COLUMN ? 4 * k + 2 : 0]), s[PER_COLUMN ? 4 * k + 2 : 0]);
        out.w = __fmul_rn(__fsub_rn(f[4 * k + 3], zf[PER_COLUMN ? 4 * k + 3 : 0]), s[PER_COLUMN ? 4 * k + 3 : 0]);
        __stcs(reinterpret_cast<float4*>(y + first) + k, out);
    }
}

template <int DX, int DZ>
__global__ void __launch_bounds__(256) dequantize_per_tensor_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, const float* __restrict__ scale,
                                                                    const void* __restrict__ zero, size_t n) {
    wait_for_previous_kernel();
    float s[1] = {__ldg(scale)};
    float zf[1] = {zero_point_value<DZ>(zero, 0)};
    const size_t runs = n / 16, step = (size_t)gridDim.x * blockDim.x;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += step) dequantize_step<DX, false>(x, y, r * 16, s, zf);
    if (blockIdx.x == 0 && threadIdx.x == 0)
        for (size_t i = runs * 16; i < n; i++) y[i] = __fmul_rn(__fsub_rn(to_f32<DX>(((const typename Storage<DX>::type*)x)[i]), zf[0]), s[0]);
}

template <int DX, int DZ>
__global__ void __launch_bounds__(256) dequantize_per_column_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, const float* __restrict__ scale,
                                                                    const void* __restrict__ zero, size_t rows, uint32_t cols) {
    wait_for_previous_kernel();
    const uint32_t groups = cols / 16;
    const size_t tid = (size_t)blockIdx.x * blockDim.x + threadIdx.x, threads = (size_t)gridDim.x * blockDim.x;
    const uint32_t col = (uint32_t)(tid % groups) * 16;
    float s[16], zf[16];
    #pragma unroll
    for (int j = 0; j < 16; j++) { s[j] = __ldg(scale + col + j); zf[j] = zero_point_value<DZ>(zero, col + j); }
    for (size_t row = tid / groups; row < rows; row += threads / groups) dequantize_step<DX, true>(x, y, row * cols + col, s, zf);
}

// ---- host ---------------------------------------------------------------------------------------------------------------
// Thread blocks of 256 such that the thread count is a multiple of `groups` (0 when that takes more than the GPU holds).
static int grid_multiple_of(uint32_t groups, size_t work_items, int sm_count) {
    uint64_t a = groups, b = 256;
    while (b) { const uint64_t t = a % b; a = b; b = t; }
    const uint64_t unit = (uint64_t)groups / a;                    // blocks per period: lcm(groups, 256) / 256
    const uint64_t limit = (uint64_t)sm_count * kEwCtasPerSm;
    if (unit > limit) return 0;
    uint64_t want = (work_items + 255) / 256;
    if (want > limit) want = limit;
    uint64_t blocks = (want / unit) * unit;
    if (blocks == 0) blocks = unit;
    return (int)blocks;
}

template <class Kernel, class... Args>
static bool launch_pdl(const char* name, Kernel kernel, int grid, Args... args) {
    static const bool overlap = [] { const char* e = getenv("TOPS_PDL"); return !(e && e[0] == '0'); }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(256);
    cfg.gridDim = dim3(grid);
    cfg.stream = current_stream();
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    check_cuda(cudaLaunchKernelEx(&cfg, kernel, args...), name);
    return TOPS_CHECK_LAUNCH(name);
}

// 0: not a case for these kernels.  1: one scale.  2: one scale per element of the last dimension.
// `s`, `z`: the shapes scale and zero point are broadcast with (after an axis attribute has been applied).
static int scale_form(const Tensor* t, const ShapeView& s, const ShapeView& z) {
    if (s.size == 1 && z.size == 1) return 1;
    if (t->ndim < 1) return 0;
    const size_t cols = (size_t)t->shape[t->ndim - 1];
    auto inner_vector = [&](const ShapeView& v) {                 // size == cols with the last dimension == cols: every other dimension is 1
        return v.size == cols && v.ndim >= 1 && v.ndim <= t->ndim && (size_t)v.shape[v.ndim - 1] == cols;
    };
    if (cols >= 16 && cols % 16 == 0 && cols <= 0x7FFFFFF0ull && inner_vector(s) && inner_vector(z)) return 2;
    return 0;
}

// Returns true when a kernel of this file took the call.
bool qdq_fast(const char* name, bool quantize, const Tensor* x, const Tensor* s, const Tensor* z, Tensor* y, const ShapeView& s_shape, const ShapeView& z_shape) {
    if (getenv("TOPS_NO_FAST_QDQ")) return false;
    const Tensor* values = quantize ? x : y;                        // the float32 side
    const Tensor* codes = quantize ? y : x;                         // the 8-bit side
    const int dc = (int)codes->dtype, dz = (int)z->dtype;
    if (values->dtype != DTYPE_FLOAT32 || s->dtype != DTYPE_FLOAT32 || x->size != y->size || y->size == 0) return false;
    const bool int_codes = dc == DTYPE_INT8 || dc == DTYPE_UINT8, fp8_codes = dc == DTYPE_FLOAT8_E4M3 || dc == DTYPE_FLOAT8_E5M2;
    if (!(int_codes && dz == dc) && !(fp8_codes && dz == DTYPE_INT8)) return false;
    if (!aligned_to(x->data, 16) || !aligned_to(y->data, 16)) return false;
    const int form = scale_form(y, s_shape, z_shape);
    if (form == 0) return false;
    DeviceState* st = acquire_device();
    if (!st) return true;
    const size_t n = y->size;
    const float* scale = (const float*)s->data;
    bool ok = true;
    if (form == 1) {
        const int grid = grid_for((n + 15) / 16, 256, st->sm_count, kEwCtasPerSm);
#define TOPS_FAST(DC, DZ)                                                                                                                  \
        if (dc == DC && dz == DZ) {                                                                                                        \
            ok = quantize ? launch_pdl(name, quantize_per_tensor_kernel<DC, DZ>, grid, (const float*)x->data, (uint8_t*)y->data, scale, (const void*)z->data, n) \
                          : launch_pdl(name, dequantize_per_tensor_kernel<DC, DZ>, grid, (const uint8_t*)x->data, (float*)y->data, scale, (const void*)z->data, n); \
        }
        TOPS_FAST(DTYPE_INT8, DTYPE_INT8) TOPS_FAST(DTYPE_UINT8, DTYPE_UINT8) TOPS_FAST(DTYPE_FLOAT8_E4M3, DTYPE_INT8) TOPS_FAST(DTYPE_FLOAT8_E5M2, DTYPE_INT8)
#undef TOPS_FAST
    } else {
        const uint32_t cols = (uint32_t)y->shape[y->ndim - 1];
        const size_t rows = n / cols;
        const int grid = grid_multiple_of(cols / 16, n / 16, st->sm_count);
        if (grid == 0) return false;
#define TOPS_FAST(DC, DZ)                                                                                                                  \
        if (dc == DC && dz == DZ) {                                                                                                        \
            ok = quantize ? launch_pdl(name, quantize_per_column_kernel<DC, DZ>, grid, (const float*)x->data, (uint8_t*)y->data, scale, (const void*)z->data, rows, cols) \
                          : launch_pdl(name, dequantize_per_column_kernel<DC, DZ>, grid, (const uint8_t*)x->data, (float*)y->data, scale, (const void*)z->data, rows, cols); \
        }
        TOPS_FAST(DTYPE_INT8, DTYPE_INT8) TOPS_FAST(DTYPE_UINT8, DTYPE_UINT8) TOPS_FAST(DTYPE_FLOAT8_E4M3, DTYPE_INT8) TOPS_FAST(DTYPE_FLOAT8_E5M2, DTYPE_INT8)
#undef TOPS_FAST
    }
    (void)ok;
    return true;
}

}  // namespace tops
