// DynamicQuantizeLinear (tensor_ops.c:3760-3809): the range [min(x, 0), max(x, 0)] of the whole tensor is
// mapped onto the codes 0..255:
//     scale = (max - min) / 255 in double (1 when that is 0),
//     zero point = round-half-away(-min / scale) clamped to 0..255,
//     y = clamp(rint(x / scale) + zero point, 0, 255), stored like any operator result.
// The division uses the DOUBLE scale; y_scale receives it rounded to its own type.
//
// Two launches and no host round trip: the first reduces x to one (min, max) pair per CTA, the second has
// every CTA fold those few hundred pairs again (they sit in L2), derive scale and zero point identically,
// and quantise its share of x; CTA 0 also writes y_scale and y_zero_point.  x is read twice -- the second
// time from L2 when it fits -- and y written once: 2 * sizeof(x) + sizeof(y) bytes per element.
#include "elementwise.cuh"
#include "qdq_math.cuh"

namespace tops {

constexpr int kDqThreads = 256;
constexpr int kDqMaxCtas = kNumSMs * 8;

// NaNs never win a comparison in the reference (v < min, v > max); fminf / fmaxf drop them the same way.
template <int DX, int V>
__global__ void __launch_bounds__(kDqThreads) range_partials_kernel(const void* __restrict__ x, size_t n, double* __restrict__ partials) {
    using S = typename Storage<DX>::type;
    constexpr bool kInFloat = dtype_exact_in_f32(DX);
    float lo_f = INFINITY, hi_f = -INFINITY;
    double lo_d = INFINITY, hi_d = -INFINITY;
    const size_t runs = n / V;
    for (size_t r = (size_t)blockIdx.x * kDqThreads + threadIdx.x; r < runs; r += (size_t)gridDim.x * kDqThreads) {
        Run<S, V> run;
        load_bytes<sizeof(S) * V>((const S*)x + r * V, &run);
        if constexpr (kInFloat) {
            float f[V];
            decode_floats<DX, V>(run, f);
            #pragma unroll
            for (int j = 0; j < V; j++) { lo_f = fminf(lo_f, f[j]); hi_f = fmaxf(hi_f, f[j]); }
        } else {
            #pragma unroll
            for (int j = 0; j < V; j++) { const double v = to_f64<DX>(run.v[j]); lo_d = fmin(lo_d, v); hi_d = fmax(hi_d, v); }
        }
    }
    if (blockIdx.x == 0)                                                     // the ragged tail
        for (size_t i = runs * V + threadIdx.x; i < n; i += kDqThreads) {
            const double v = to_f64<DX>(((const S*)x)[i]);
            lo_d = fmin(lo_d, v); hi_d = fmax(hi_d, v);
        }
    if constexpr (kInFloat) { lo_d = fmin(lo_d, (double)lo_f); hi_d = fmax(hi_d, (double)hi_f); }
    #pragma unroll
    for (int o = 16; o; o >>= 1) { lo_d = fmin(lo_d, __shfl_xor_sync(0xFFFFFFFFu, lo_d, o)); hi_d = fmax(hi_d, __shfl_xor_sync(0xFFFFFFFFu, hi_d, o)); }
    __shared__ double s_lo[kDqThreads / 32], s_hi[kDqThreads / 32];
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo_d; s_hi[threadIdx.x >> 5] = hi_d; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kDqThreads / 32; w++) { lo_d = fmin(lo_d, s_lo[w]); hi_d = fmax(hi_d, s_hi[w]); }
        partials[2 * blockIdx.x] = lo_d;
        partials[2 * blockIdx.x + 1] = hi_d;
    }
}

// Runtime-typed variant for the remaining input types.
__global__ void __launch_bounds__(kDqThreads) range_partials_generic(const void* __restrict__ x, int dx, size_t n, double* __restrict__ partials) {
    double lo = INFINITY, hi = -INFINITY;
    for (size_t i = (size_t)blockIdx.x * kDqThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kDqThreads) {
        const double v = load_f64_rt(x, dx, i);
        lo = fmin(lo, v); hi = fmax(hi, v);
    }
    #pragma unroll
    for (int o = 16; o; o >>= 1) { lo = fmin(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o)); hi = fmax(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o)); }
    __shared__ double s_lo[kDqThreads / 32], s_hi[kDqThreads / 32];
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kDqThreads / 32; w++) { lo = fmin(lo, s_lo[w]); hi = fmax(hi, s_hi[w]); }
        partials[2 * blockIdx.x] = lo;
        partials[2 * blockIdx.x + 1] = hi;
    }
}

struct DynamicScale { double scale; double zero; };

// Every thread of the CTA returns the same pair; CTA 0 publishes it.
__device__ __forceinline__ DynamicScale fold_range(const double* __restrict__ partials, int n_partials, void* y_scale, int ds, void* y_zero, int dz) {
    double lo = INFINITY, hi = -INFINITY;
    for (int i = threadIdx.x; i < n_partials; i += kDqThreads) { lo = fmin(lo, partials[2 * i]); hi = fmax(hi, partials[2 * i + 1]); }
    #pragma unroll
    for (int o = 16; o; o >>= 1) { lo = fmin(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o)); hi = fmax(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o)); }
    __shared__ double s_lo[kDqThreads / 32], s_hi[kDqThreads / 32];
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    lo = s_lo[0]; hi = s_hi[0];
    #pragma unroll
    for (int w = 1; w < kDqThreads / 32; w++) { lo = fmin(lo, s_lo[w]); hi = fmax(hi, s_hi[w]); }
    lo = fmin(lo, 0.0);                  // also turns the "nothing seen" +-Inf into 0, as the reference's DBL_MAX start does
    hi = fmax(hi, 0.0);
    DynamicScale r;
    r.scale = __ddiv_rn(__dsub_rn(hi, lo), 255.0);
    if (r.scale == 0.0) r.scale = 1.0;
    double z = round(__dsub_rn(0.0, __ddiv_rn(lo, r.scale)));
    if (z < 0.0) z = 0.0;
    if (z > 255.0) z = 255.0;
    if (!(z == z)) z = 0.0;              // infinite range: the reference's narrowing cast of a NaN yields 0
    r.zero = z;
    if (blockIdx.x == 0 && threadIdx.x == 0) {
        store_f64_rt(y_scale, ds, 0, r.scale);
        store_f64_rt(y_zero, dz, 0, z);
    }
    return r;
}

// float32-exact inputs, uint8 codes: the rounding of qdq_math.cuh with the reciprocal of the float-rounded
// scale (its error stays inside that fast path's margin); inconclusive elements divide by the double scale.
template <int DX, int V>
__global__ void __launch_bounds__(kDqThreads) dynamic_quantize_kernel(const void* __restrict__ x, uint8_t* __restrict__ y, size_t n,
                                                                      const double* __restrict__ partials, int n_partials,
                                                                      void* y_scale, int ds, void* y_zero, int dz) {
    using S = typename Storage<DX>::type;
    const DynamicScale q = fold_range(partials, n_partials, y_scale, ds, y_zero, dz);
    const float inv = quantize_reciprocal((float)q.scale);
    const int z = (int)q.zero;
    const int z_minus_magic = z - 0x4B400000;
    const size_t runs = n / V;
    for (size_t r = (size_t)blockIdx.x * kDqThreads + threadIdx.x; r < runs; r += (size_t)gridDim.x * kDqThreads) {
        const size_t at = runs - 1 - r;          // backwards: the end of x is what the range pass left in L2
        Run<S, V> run;
        load_bytes_stream<sizeof(S) * V>((const S*)x + at * V, &run);
        float f[V];
        decode_floats<DX, V>(run, f);
        int v[V];
        bool all_ok = true;
        #pragma unroll
        for (int j = 0; j < V; j++) { bool ok; v[j] = quantize_round_8bit(f[j], inv, z_minus_magic, ok); all_ok = all_ok && ok; }
        if (!all_ok) {
            #pragma unroll
            for (int j = 0; j < V; j++) {
                double t = __dadd_rn(rint(__ddiv_rn((double)f[j], q.scale)), q.zero);
                t = t < 0.0 ? 0.0 : t;
                t = t > 255.0 ? 255.0 : t;
                v[j] = (int)from_f64<DTYPE_UINT8>(t);             // NaN passes both comparisons, as in the reference
            }
        }
        Run<typename Storage<DTYPE_UINT8>::type, V> out;
        encode_ints<DTYPE_UINT8, V>(v, out);
        store_bytes_stream<V>(y + at * V, &out);
    }
    if (blockIdx.x == 0)
        for (size_t i = runs * V + threadIdx.x; i < n; i += kDqThreads) {
            double t = __dadd_rn(rint(__ddiv_rn(to_f64<DX>(((const S*)x)[i]), q.scale)), q.zero);
            t = t < 0.0 ? 0.0 : t;
            t = t > 255.0 ? 255.0 : t;
            y[i] = from_f64<DTYPE_UINT8>(t);
        }
}

__global__ void __launch_bounds__(kDqThreads) dynamic_quantize_generic(const void* __restrict__ x, int dx, void* __restrict__ y, int dy, size_t n,
                                                                       const double* __restrict__ partials, int n_partials,
                                                                       void* y_scale, int ds, void* y_zero, int dz) {
    const DynamicScale q = fold_range(partials, n_partials, y_scale, ds, y_zero, dz);
    for (size_t i = (size_t)blockIdx.x * kDqThreads + threadIdx.x; i < n; i += (size_t)gridDim.x * kDqThreads) {
        double t = __dadd_rn(rint(__ddiv_rn(load_f64_rt(x, dx, i), q.scale)), q.zero);
        t = t < 0.0 ? 0.0 : t;
        t = t > 255.0 ? 255.0 : t;
        store_f64_rt(y, dy, i, t);
    }
}

// Folds the per-CTA pairs into range[0] = min, range[1] = max (no clamping to 0 yet: ranges of several
// shards are combined first).
__global__ void __launch_bounds__(kDqThreads) fold_partials_kernel(const double* __restrict__ partials, int n_partials, double* __restrict__ range) {
    double lo = INFINITY, hi = -INFINITY;
    for (int i = threadIdx.x; i < n_partials; i += kDqThreads) { lo = fmin(lo, partials[2 * i]); hi = fmax(hi, partials[2 * i + 1]); }
    #pragma unroll
    for (int o = 16; o; o >>= 1) { lo = fmin(lo, __shfl_xor_sync(0xFFFFFFFFu, lo, o)); hi = fmax(hi, __shfl_xor_sync(0xFFFFFFFFu, hi, o)); }
    __shared__ double s_lo[kDqThreads / 32], s_hi[kDqThreads / 32];
    if ((threadIdx.x & 31) == 0) { s_lo[threadIdx.x >> 5] = lo; s_hi[threadIdx.x >> 5] = hi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < kDqThreads / 32; w++) { lo = fmin(lo, s_lo[w]); hi = fmax(hi, s_hi[w]); }
        range[0] = lo;
        range[1] = hi;
    }
}

static int dq_ctas(size_t n) {
    const size_t per_cta = (size_t)kDqThreads * 16;
    const size_t want = (n + per_cta - 1) / per_cta;
    return (int)(want < 1 ? 1 : (want > (size_t)kDqMaxCtas ? (size_t)kDqMaxCtas : want));
}

static void launch_range(const Tensor* x, double* partials, int ctas, cudaStream_t s) {
    const int dx = (int)x->dtype;
    const bool aligned = ((uintptr_t)x->data & 15) == 0;
    if (aligned && dx == DTYPE_FLOAT32) range_partials_kernel<DTYPE_FLOAT32, 16><<<ctas, kDqThreads, 0, s>>>(x->data, x->size, partials);
    else if (aligned && dx == DTYPE_FLOAT16) range_partials_kernel<DTYPE_FLOAT16, 16><<<ctas, kDqThreads, 0, s>>>(x->data, x->size, partials);
    else if (aligned && dx == DTYPE_BFLOAT16) range_partials_kernel<DTYPE_BFLOAT16, 16><<<ctas, kDqThreads, 0, s>>>(x->data, x->size, partials);
    else range_partials_generic<<<ctas, kDqThreads, 0, s>>>(x->data, dx, x->size, partials);
}

static void launch_quantise(const Tensor* x, Tensor* y, Tensor* y_scale, Tensor* y_zp, const double* partials, int n_partials, int ctas, cudaStream_t s) {
    const int dx = (int)x->dtype, dy = (int)y->dtype, ds = (int)y_scale->dtype, dz = (int)y_zp->dtype;
    const bool fast = dy == DTYPE_UINT8 && (((uintptr_t)x->data | (uintptr_t)y->data) & 15) == 0;
    if (fast && dx == DTYPE_FLOAT32) dynamic_quantize_kernel<DTYPE_FLOAT32, 16><<<ctas, kDqThreads, 0, s>>>(x->data, (uint8_t*)y->data, x->size, partials, n_partials, y_scale->data, ds, y_zp->data, dz);
    else if (fast && dx == DTYPE_FLOAT16) dynamic_quantize_kernel<DTYPE_FLOAT16, 16><<<ctas, kDqThreads, 0, s>>>(x->data, (uint8_t*)y->data, x->size, partials, n_partials, y_scale->data, ds, y_zp->data, dz);
    else if (fast && dx == DTYPE_BFLOAT16) dynamic_quantize_kernel<DTYPE_BFLOAT16, 16><<<ctas, kDqThreads, 0, s>>>(x->data, (uint8_t*)y->data, x->size, partials, n_partials, y_scale->data, ds, y_zp->data, dz);
    else dynamic_quantize_generic<<<ctas, kDqThreads, 0, s>>>(x->data, dx, y->data, dy, x->size, partials, n_partials, y_scale->data, ds, y_zp->data, dz);
}

static bool dq_outputs_ok(const char* name, const Tensor* x, Tensor* y, Tensor* y_scale, Tensor* y_zp) {
    if (!x || !y || !y_scale || !y_zp || !y_scale->data || !y_zp->data || (x->size && (!x->data || !y->data)) || x->size != y->size ||
        y_scale->size < 1 || y_zp->size < 1) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor, size mismatch or empty scale / zero point", name);
        zero_fill(y);
        return false;
    }
    if (!dtype_valid((int)x->dtype) || !dtype_valid((int)y->dtype) || !dtype_valid((int)y_scale->dtype) || !dtype_valid((int)y_zp->dtype)) {
        set_error(TOPS_ERR_INVALID, "%s: bad dtype", name);
        return false;
    }
    return true;
}

}  // namespace tops

using namespace tops;

TOPS_API void dynamic_quantize_linear_forward(const Tensor* x, Tensor* y, Tensor* y_scale, Tensor* y_zp) {
    const char* name = "dynamic_quantize_linear_forward";
    if (!dq_outputs_ok(name, x, y, y_scale, y_zp)) return;
    DeviceState* st = acquire_device();
    if (!st) return;
    cudaStream_t s = current_stream();
    const int ctas = dq_ctas(x->size);
    double* partials = nullptr;
    if (cudaMallocAsync((void**)&partials, sizeof(double) * 2 * (size_t)ctas, s) != cudaSuccess) { cudaGetLastError(); set_error(TOPS_ERR_OOM, "%s: scratch", name); return; }
    launch_range(x, partials, ctas, s);
    launch_quantise(x, y, y_scale, y_zp, partials, ctas, ctas, s);
    TOPS_CHECK_LAUNCH(name);
    cudaFreeAsync(partials, s);
    finish_op();
}

TOPS_API int tops_dynamic_quantize_range(const Tensor* x, Tensor* range) {
    const char* name = "tops_dynamic_quantize_range";
    if (!x || !range || !range->data || range->size < 2 || (int)range->dtype != DTYPE_FLOAT64 || (x->size && !x->data) || !dtype_valid((int)x->dtype)) {
        set_error(TOPS_ERR_INVALID, "%s: wants a tensor and a float64 range of two elements", name);
        return tops_last_error();
    }
    DeviceState* st = acquire_device();
    if (!st) return tops_last_error();
    cudaStream_t s = current_stream();
    const int ctas = dq_ctas(x->size);
    double* partials = nullptr;
    if (cudaMallocAsync((void**)&partials, sizeof(double) * 2 * (size_t)ctas, s) != cudaSuccess) { cudaGetLastError(); set_error(TOPS_ERR_OOM, "%s: scratch", name); return tops_last_error(); }
    launch_range(x, partials, ctas, s);
    fold_partials_kernel<<<1, kDqThreads, 0, s>>>(partials, ctas, (double*)range->data);
    TOPS_CHECK_LAUNCH(name);
    cudaFreeAsync(partials, s);
    finish_op();
    return tops_last_error();
}

TOPS_API int tops_dynamic_quantize_apply(const Tensor* x, const Tensor* range, Tensor* y, Tensor* y_scale, Tensor* y_zp) {
    const char* name = "tops_dynamic_quantize_apply";
    if (!range || !range->data || range->size < 2 || (int)range->dtype != DTYPE_FLOAT64) {
        set_error(TOPS_ERR_INVALID, "%s: wants a float64 range of two elements", name);
        zero_fill(y);
        return tops_last_error();
    }
    if (!dq_outputs_ok(name, x, y, y_scale, y_zp)) return tops_last_error();
    DeviceState* st = acquire_device();
    if (!st) return tops_last_error();
    launch_quantise(x, y, y_scale, y_zp, (const double*)range->data, 1, dq_ctas(x->size), current_stream());
    TOPS_CHECK_LAUNCH(name);
    finish_op();
    return tops_last_error();
}
