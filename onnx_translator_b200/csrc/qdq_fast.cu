// QuantizeLinear / DequantizeLinear (tensor_ops.c:999-1034) for the two shapes of scale that dominate real graphs,
// written as loops a thread stays in: float32 values against 8-bit codes with
//   * one scale and one zero point for the whole tensor, or
//   * one per element of the innermost dimension (per-axis on the last axis).
// Everything that does not depend on the element -- reciprocal of the scale, zero point folded into the rounding
// constant -- is computed once per thread instead of once per run, and a thread moves 16 elements per step, as four
// groups of four that interleave with the other lanes' groups so that each instruction of the warp is one contiguous
// span.  The arithmetic is that of the general bodies (qdq_math.cuh): rounding by adding 1.5 * 2^23, a tie margin test,
// the reference's double division for the rare undecided group.
// For the per-axis form the grid is sized so that a warp meets the same 128 columns on every step.
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

// A warp works on tiles; inside a tile lane l owns the groups of four consecutive elements l, l + 32, l + 64, l + 96, so
// every load and every store instruction of the warp covers one contiguous span (512 bytes of float32, 128 bytes of
// codes) -- a thread that walked 16 consecutive elements would write each 32-byte sector in two halves.

// Four values -> four codes in one word.  Returns false when the fast rounding could not decide some element.
template <int DO>
__device__ __forceinline__ bool quantize4(const float4 x, const float (&inv)[4], const float (&zt)[4], uint32_t& word) {
    constexpr bool kFp8 = DO == DTYPE_FLOAT8_E4M3 || DO == DTYPE_FLOAT8_E5M2;
    const float v[4] = {x.x, x.y, x.z, x.w};
    bool all_ok = true;
    if constexpr (kFp8) {
        float fr[4];
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            const float q = __fmul_rn(v[j], inv[j]);
            const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
            all_ok = all_ok & (fmaf(fabsf(q), 1.9073486e-6f, fabsf(__fsub_rn(q, rq))) < 0.5f);
            if constexpr (DO == DTYPE_FLOAT8_E5M2) all_ok = all_ok & (fabsf(q) < 57000.0f);     // beyond: the reference overflows to infinity
            fr[j] = __fadd_rn(rq, zt[j]);
        }
        const uint32_t lo = __nv_cvt_float2_to_fp8x2(make_float2(fr[0], fr[1]), __NV_SATFINITE, DO == DTYPE_FLOAT8_E4M3 ? __NV_E4M3 : __NV_E5M2);
        const uint32_t hi = __nv_cvt_float2_to_fp8x2(make_float2(fr[2], fr[3]), __NV_SATFINITE, DO == DTYPE_FLOAT8_E4M3 ? __NV_E4M3 : __NV_E5M2);
        word = lo | (hi << 16);
    } else {
        int c[4];
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            const float q = __fmul_rn(v[j], inv[j]);
            const float t = __fadd_rn(q, 12582912.0f);
            const float d = __fsub_rn(q, __fsub_rn(t, 12582912.0f));
            all_ok = all_ok & (fmaf(fabsf(q), 1.9073486e-6f, fabsf(d)) < 0.5f);
            c[j] = __float_as_int(t) + __float_as_int(zt[j]);
        }
        word = DO == DTYPE_INT8 ? pack_sat_s8x4(c[0], c[1], c[2], c[3]) : pack_sat_u8x4(c[0], c[1], c[2], c[3]);
    }
    return all_ok;
}

// Quantise four groups of four elements (16-byte aligned, at first[k]; `on[k]` false skips a group).  All four loads are
// issued before the first value is used.  `col`: index of a group's first scale / zero point, `col_step` 1 when the
// scales differ per column, 0 when one scale serves all.
template <int DO, int DZ>
__device__ __forceinline__ void quantize_groups(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                                const void* __restrict__ zero, const size_t (&first)[4], const bool (&on)[4], size_t col,
                                                size_t col_step, const float (&inv)[4], const float (&zt)[4]) {
    float4 v[4];
    #pragma unroll
    for (int k = 0; k < 4; k++) v[k] = on[k] ? __ldcs(reinterpret_cast<const float4*>(x + first[k])) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    uint32_t word[4];
    bool ok[4];
    #pragma unroll
    for (int k = 0; k < 4; k++) ok[k] = quantize4<DO>(v[k], inv, zt, word[k]);
    #pragma unroll
    for (int k = 0; k < 4; k++) {
        if (!on[k]) continue;
        if (!ok[k]) {                                                // rare: a rounding tie, a huge or a non-finite value
            const float e[4] = {v[k].x, v[k].y, v[k].z, v[k].w};
            word[k] = 0;
            #pragma unroll
            for (int j = 0; j < 4; j++) {
                const size_t c = col + j * col_step;
                word[k] |= quantize_exact_code<DO>(e[j], scale[c], zero_point_value<DZ>(zero, c)) << (8 * j);
            }
        }
        __stcs(reinterpret_cast<uint32_t*>(y + first[k]), word[k]);
    }
}

constexpr int kTileElems = 512;          // per warp and step: 4 groups of 4 elements per lane

template <int DO, int DZ>
__global__ void __launch_bounds__(256) quantize_per_tensor_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                                                  const void* __restrict__ zero, size_t n) {
    wait_for_previous_kernel();
    const float inv1 = quantize_reciprocal(__ldg(scale)), zt1 = zero_point_term<DO, DZ>(zero, 0);
    const float inv[4] = {inv1, inv1, inv1, inv1}, zt[4] = {zt1, zt1, zt1, zt1};
    const size_t lane = threadIdx.x & 31, warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t tiles = n / kTileElems;
    const bool on[4] = {true, true, true, true};
    for (size_t t = warp; t < tiles; t += warps) {
        const size_t base = t * kTileElems + lane * 4;
        const size_t first[4] = {base, base + 128, base + 256, base + 384};
        quantize_groups<DO, DZ>(x, y, scale, zero, first, on, 0, 0, inv, zt);
    }
    if (warp == 0)                                                   // what does not fill a tile: element by element, the reference's way
        for (size_t i = tiles * kTileElems + lane; i < n; i += 32) y[i] = (uint8_t)quantize_exact_code<DO>(x[i], scale[0], zero_point_value<DZ>(zero, 0));
}

// rows x cols with scale / zero of length cols; cols is a multiple of 128.  A warp owns one tile of 128 columns (lane l
// the columns 4l .. 4l + 3 of it, whose reciprocals and zero points it keeps) and walks down the rows four at a time;
// the warp count is a multiple of the number of column tiles.
template <int DO, int DZ>
__global__ void __launch_bounds__(256) quantize_per_column_kernel(const float* __restrict__ x, uint8_t* __restrict__ y, const float* __restrict__ scale,
                                                                  const void* __restrict__ zero, size_t rows, uint32_t cols) {
    wait_for_previous_kernel();
    const uint32_t col_tiles = cols / 128;
    const size_t lane = threadIdx.x & 31, warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t col = (warp % col_tiles) * 128 + lane * 4;
    float inv[4], zt[4];
    #pragma unroll
    for (int j = 0; j < 4; j++) { inv[j] = quantize_reciprocal(__ldg(scale + col + j)); zt[j] = zero_point_term<DO, DZ>(zero, col + j); }
    for (size_t row = (warp / col_tiles) * 4; row < rows; row += (warps / col_tiles) * 4) {
        const size_t base = row * cols + col;
        const size_t first[4] = {base, base + cols, base + 2 * (size_t)cols, base + 3 * (size_t)cols};
        const bool on[4] = {true, row + 1 < rows, row + 2 < rows, row + 3 < rows};
        quantize_groups<DO, DZ>(x, y, scale, zero, first, on, col, 1, inv, zt);
    }
}

// ---- Dequantize: four codes (one word) -> four float32 ---------------------------------------------------------------------
template <int DX>
__device__ __forceinline__ void dequantize_word(uint32_t w, float* __restrict__ dst, const float (&s)[4], const float (&zf)[4]) {
    float f[4];
    if constexpr (DX == DTYPE_INT8 || DX == DTYPE_UINT8) {
        // the byte becomes the low mantissa byte of 2^23 (signed bytes biased by 128 first), then the bias is subtracted
        const uint32_t word = DX == DTYPE_INT8 ? (w ^ 0x80808080u) : w;
        const float bias = DX == DTYPE_INT8 ? 8388736.0f : 8388608.0f;
        f[0] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540)), bias);
        f[1] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7541)), bias);
        f[2] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7542)), bias);
        f[3] = __fsub_rn(__uint_as_float(__byte_perm(word, 0x4B000000u, 0x7543)), bias);
    } else {
        #pragma unroll
        for (int h = 0; h < 2; h++) {                                // two float8 codes per hardware convert
            const uint16_t two = (uint16_t)(w >> (16 * h));
            uint32_t half2_bits;
            if constexpr (DX == DTYPE_FLOAT8_E4M3) {
                const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(two, __NV_E4M3);
                half2_bits = (uint32_t)hr.x | ((uint32_t)hr.y << 16);
            } else {
                half2_bits = __byte_perm((uint32_t)two, 0u, 0x1404);   // an e5m2 code is the upper byte of a float16
            }
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&half2_bits));
            f[2 * h] = p.x; f[2 * h + 1] = p.y;
        }
    }
    float4 out;
    out.x = __fmul_rn(__fsub_rn(f[0], zf[0]), s[0]);
    out.y = __fmul_rn(__fsub_rn(f[1], zf[1]), s[1]);
    out.z = __fmul_rn(__fsub_rn(f[2], zf[2]), s[2]);
    out.w = __fmul_rn(__fsub_rn(f[3], zf[3]), s[3]);
    __stcs(reinterpret_cast<float4*>(dst), out);
}

// Four groups of four codes (one word each, at first[k]); all four loads are issued before the first is used.
template <int DX>
__device__ __forceinline__ void dequantize_groups(const uint8_t* __restrict__ x, float* __restrict__ y, const size_t (&first)[4], const bool (&on)[4],
                                                  const float (&s)[4], const float (&zf)[4]) {
    uint32_t w[4];
    #pragma unroll
    for (int k = 0; k < 4; k++) w[k] = on[k] ? __ldcs(reinterpret_cast<const uint32_t*>(x + first[k])) : 0u;
    #pragma unroll
    for (int k = 0; k < 4; k++) if (on[k]) dequantize_word<DX>(w[k], y + first[k], s, zf);
}

template <int DX, int DZ>
__global__ void __launch_bounds__(256) dequantize_per_tensor_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, const float* __restrict__ scale,
                                                                    const void* __restrict__ zero, size_t n) {
    wait_for_previous_kernel();
    const float s1 = __ldg(scale), z1 = zero_point_value<DZ>(zero, 0);
    const float s[4] = {s1, s1, s1, s1}, zf[4] = {z1, z1, z1, z1};
    const size_t lane = threadIdx.x & 31, warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t tiles = n / kTileElems;
    const bool on[4] = {true, true, true, true};
    for (size_t t = warp; t < tiles; t += warps) {
        const size_t base = t * kTileElems + lane * 4;
        const size_t first[4] = {base, base + 128, base + 256, base + 384};
        dequantize_groups<DX>(x, y, first, on, s, zf);
    }
    if (warp == 0)
        for (size_t i = tiles * kTileElems + lane; i < n; i += 32)
            y[i] = __fmul_rn(__fsub_rn(to_f32<DX>(((const typename Storage<DX>::type*)x)[i]), z1), s1);
}

template <int DX, int DZ>
__global__ void __launch_bounds__(256) dequantize_per_column_kernel(const uint8_t* __restrict__ x, float* __restrict__ y, const float* __restrict__ scale,
                                                                    const void* __restrict__ zero, size_t rows, uint32_t cols) {
    wait_for_previous_kernel();
    const uint32_t col_tiles = cols / 128;
    const size_t lane = threadIdx.x & 31, warp = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = ((size_t)gridDim.x * blockDim.x) >> 5;
    const size_t col = (warp % col_tiles) * 128 + lane * 4;
    float s[4], zf[4];
    #pragma unroll
    for (int j = 0; j < 4; j++) { s[j] = __ldg(scale + col + j); zf[j] = zero_point_value<DZ>(zero, col + j); }
    for (size_t row = (warp / col_tiles) * 4; row < rows; row += (warps / col_tiles) * 4) {
        const size_t base = row * cols + col;
        const size_t first[4] = {base, base + cols, base + 2 * (size_t)cols, base + 3 * (size_t)cols};
        const bool on[4] = {true, row + 1 < rows, row + 2 < rows, row + 3 < rows};
        dequantize_groups<DX>(x, y, first, on, s, zf);
    }
}

// ---- host ---------------------------------------------------------------------------------------------------------------
// Thread blocks of 256 (8 warps) such that the warp count is a multiple of `groups` (0 when that takes more than the GPU holds).
static int grid_multiple_of(uint32_t groups, size_t work_items, int sm_count) {
    uint64_t a = groups, b = 8;
    while (b) { const uint64_t t = a % b; a = b; b = t; }
    const uint64_t unit = (uint64_t)groups / a;                    // blocks per period: lcm(groups, 8) / 8
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
    if (cols >= 128 && cols % 128 == 0 && cols <= 0x7FFFFF80ull && inner_vector(s) && inner_vector(z)) return 2;
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
        const int grid = grid_for((n + 15) / 16, 256, st->sm_count, kEwCtasPerSm);       // 16 elements per thread and step
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
        const int grid = grid_multiple_of(cols / 128, n / 16, st->sm_count);
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
