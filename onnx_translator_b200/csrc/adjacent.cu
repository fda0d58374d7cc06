// Operators that surround the hot path in exported convolutional networks: Clip, AveragePool,
// GlobalAveragePool and BatchNormalization (tensor_ops.c:1523-1543, 2735-2789, 2844-2868, 3041-3083).
// All arithmetic is the reference's, in double and in its order, so the outputs are bit-identical:
// the generic kernels are one thread per output (or per plane) with the dtypes switched at run time; float32 /
// float16 / bfloat16 tensors take typed variants with vector accesses.
#include "elementwise.cuh"

namespace tops {

// ---- Clip ---------------------------------------------------------------------------------------------------
// Compare in double, lower bound first; a NaN value or bound changes nothing.  Bounds are optional and
// broadcast against the input (the reference's caller materialises them at full size).
struct ClipArgs {
    Geometry g;
    Operand x, lo, hi;
    int dx, dlo, dhi, dout, has_lo, has_hi;
};

__global__ void __launch_bounds__(256) clip_kernel(ClipArgs a, void* __restrict__ y, size_t first, uint32_t n) {
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        uint32_t p;
        double v = load_f64_rt(a.x.ptr, a.dx, a.x.flat ? i : operand_offset(a.g, a.x, i, p));
        if (a.has_lo) { const double b = load_f64_rt(a.lo.ptr, a.dlo, a.lo.flat ? i : operand_offset(a.g, a.lo, i, p)); if (v < b) v = b; }
        if (a.has_hi) { const double b = load_f64_rt(a.hi.ptr, a.dhi, a.hi.flat ? i : operand_offset(a.g, a.hi, i, p)); if (v > b) v = b; }
        store_f64_rt(y, a.dout, first + i, v);
    }
}

// Same float type in and out, scalar bounds whose values are exact in float32: the comparisons give the same
// answers in float32 as in double, and the stored value is the input or a bound either way.
template <int DT>
__global__ void __launch_bounds__(256) clip_typed_kernel(const void* __restrict__ x, void* __restrict__ y, size_t n, const void* lo, int dlo,
                                                         const void* hi, int dhi) {
    using S = typename Storage<DT>::type;
    constexpr int V = 16 / (int)sizeof(S);
    const bool has_lo = lo != nullptr, has_hi = hi != nullptr;
    const float lof = has_lo ? (float)load_f64_rt(lo, dlo, 0) : 0.0f, hif = has_hi ? (float)load_f64_rt(hi, dhi, 0) : 0.0f;
    const size_t runs = n / V;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += (size_t)gridDim.x * blockDim.x) {
        Run<S, V> in, out;
        load_bytes_stream<16>((const S*)x + r * V, &in);
        float f[V];
        decode_floats<DT, V>(in, f);
        #pragma unroll
        for (int j = 0; j < V; j++) {
            if (has_lo && f[j] < lof) f[j] = lof;
            if (has_hi && f[j] > hif) f[j] = hif;
        }
        encode_floats<DT, V>(f, out);
        store_bytes_stream<16>((S*)y + r * V, &out);
    }
    if (blockIdx.x == 0)
        for (size_t i = runs * V + threadIdx.x; i < n; i += blockDim.x) {
            float v = to_f32<DT>(((const S*)x)[i]);
            if (has_lo && v < lof) v = lof;
            if (has_hi && v > hif) v = hif;
            ((S*)y)[i] = from_f32<DT>(v);
        }
}

// ---- AveragePool --------------------------------------------------------------------------------------------
struct AvgGeom {
    int C, H, W, OH, OW, KH, KW, pt, pl, sh, sw, dh, dw, include_pad;
};

__global__ void __launch_bounds__(256) average_pool_kernel(const void* __restrict__ x, void* __restrict__ y, int dx, int dout,
                                                           AvgGeom p, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ow = (int)(i % (size_t)p.OW);
        const size_t t = i / (size_t)p.OW;
        const int oh = (int)(t % (size_t)p.OH);
        const size_t in_base = (t / (size_t)p.OH) * (size_t)p.H * (size_t)p.W;
        double sum = 0.0;
        int count = 0;
        for (int kh = 0; kh < p.KH; kh++) {
            const int ih = oh * p.sh + kh * p.dh - p.pt;
            for (int kw = 0; kw < p.KW; kw++) {
                const int iw = ow * p.sw + kw * p.dw - p.pl;
                if (ih < 0 || ih >= p.H || iw < 0 || iw >= p.W) { count += p.include_pad; continue; }
                sum = __dadd_rn(sum, load_f64_rt(x, dx, in_base + (size_t)ih * p.W + iw));      // kh -> kw order, as the reference
                count++;
            }
        }
        store_f64_rt(y, dout, i, count > 0 ? __ddiv_rn(sum, (double)count) : 0.0);
    }
}

// ---- GlobalAveragePool -----------------------------------------------------------------------------------------
// One thread per H x W plane, adding in the reference's sequential order (a parallel sum would round
// differently).  Neighbouring threads read neighbouring planes, i.e. addresses `spatial` elements apart; each
// thread's own stream is contiguous, so the cache lines it touches are reused by its next iterations.
__global__ void __launch_bounds__(128) global_average_pool_kernel(const void* __restrict__ x, void* __restrict__ y, int dx, int dout,
                                                                  size_t planes, int spatial) {
    for (size_t n = (size_t)blockIdx.x * blockDim.x + threadIdx.x; n < planes; n += (size_t)gridDim.x * blockDim.x) {
        double sum = 0.0;
        const size_t base = n * (size_t)spatial;
        for (int i = 0; i < spatial; i++) sum = __dadd_rn(sum, load_f64_rt(x, dx, base + i));
        store_f64_rt(y, dout, n, __ddiv_rn(sum, (double)spatial));
    }
}

// float32 / float16 / bfloat16 planes: a warp takes 8 planes at a time.  All 32 lanes fetch 128 consecutive
// elements of each plane with coalesced loads into shared memory, then lanes 0..7 each add their own plane's
// 128 values in order -- the chain of dependent additions is the reference's, the memory accesses are not.
constexpr int kGapPlanes = 8, kGapChunk = 128, kGapWarps = 4;

template <int DT>
__global__ void __launch_bounds__(kGapWarps * 32) global_average_pool_typed(const void* __restrict__ x, void* __restrict__ y, int dout,
                                                                             size_t planes, int spatial) {
    using S = typename Storage<DT>::type;
    __shared__ double tile[kGapWarps][kGapPlanes][kGapChunk + 1];     // widened by all 32 lanes, so the adding lanes only load and add
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t groups = (planes + kGapPlanes - 1) / kGapPlanes;
    for (size_t grp = (size_t)blockIdx.x * kGapWarps + warp; grp < groups; grp += (size_t)gridDim.x * kGapWarps) {
        const size_t p0 = grp * kGapPlanes;
        double sum = 0.0;
        float v[kGapPlanes][kGapChunk / 32];
        auto fetch = [&](int c0) {
            #pragma unroll
            for (int r = 0; r < kGapPlanes; r++)
                #pragma unroll
                for (int q = 0; q < kGapChunk / 32; q++) {
                    const int c = c0 + q * 32 + lane;
                    v[r][q] = (p0 + r < planes && c < spatial) ? to_f32<DT>(((const S*)x)[(p0 + r) * (size_t)spatial + c]) : 0.0f;
                }
        };
        fetch(0);
        for (int c0 = 0; c0 < spatial; c0 += kGapChunk) {
            #pragma unroll
            for (int r = 0; r < kGapPlanes; r++)
                #pragma unroll
                for (int q = 0; q < kGapChunk / 32; q++) tile[warp][r][q * 32 + lane] = (double)v[r][q];
            __syncwarp();
            if (c0 + kGapChunk < spatial) fetch(c0 + kGapChunk);          // in flight while this chunk is added up
            if (lane < kGapPlanes) {
                const int m = spatial - c0 < kGapChunk ? spatial - c0 : kGapChunk;
                for (int j = 0; j < m; j++) sum = __dadd_rn(sum, tile[warp][lane][j]);
            }
            __syncwarp();
        }
        if (lane < kGapPlanes && p0 + lane < planes) store_f64_rt(y, dout, p0 + lane, __ddiv_rn(sum, (double)spatial));
    }
}

// ---- BatchNormalization (inference) ------------------------------------------------------------------------------
// Per channel a = scale / sqrt(var + eps), k = bias - mean * a (a small kernel fills the two tables), then
// y = x * a + k with the product and the sum rounded separately.
__global__ void batch_norm_tables(const void* scale, const void* bias, const void* mean, const void* var, int ds, int db, int dm, int dv,
                                  double epsilon, int C, double* __restrict__ a, double* __restrict__ k) {
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    const double inv_std = __ddiv_rn(1.0, sqrt(__dadd_rn(load_f64_rt(var, dv, c), epsilon)));
    const double av = __dmul_rn(load_f64_rt(scale, ds, c), inv_std);
    a[c] = av;
    k[c] = __dsub_rn(load_f64_rt(bias, db, c), __dmul_rn(load_f64_rt(mean, dm, c), av));
}

__global__ void __launch_bounds__(256) batch_norm_kernel(const void* __restrict__ x, void* __restrict__ y, int dx, int dout, int C,
                                                         uint32_t spatial, const double* __restrict__ a, const double* __restrict__ k,
                                                         size_t first_plane) {
    const size_t plane = first_plane + blockIdx.y;                   // n * C + c
    const double av = a[plane % (size_t)C], kv = k[plane % (size_t)C];
    const size_t base = plane * (size_t)spatial;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < spatial; i += gridDim.x * blockDim.x)
        store_f64_rt(y, dout, base + i, __dadd_rn(__dmul_rn(load_f64_rt(x, dx, base + i), av), kv));
}

// Same float type in and out, plane size a multiple of the vector width: vector accesses, the arithmetic unchanged.
template <int DT>
__global__ void __launch_bounds__(256) batch_norm_typed_kernel(const void* __restrict__ x, void* __restrict__ y, int C, uint32_t spatial,
                                                               const double* __restrict__ a, const double* __restrict__ k, size_t first_plane) {
    using S = typename Storage<DT>::type;
    constexpr int V = 16 / (int)sizeof(S);
    const size_t plane = first_plane + blockIdx.y;
    const double av = a[plane % (size_t)C], kv = k[plane % (size_t)C];
    const S* xp = (const S*)x + plane * (size_t)spatial;
    S* yp = (S*)y + plane * (size_t)spatial;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < spatial / V; r += gridDim.x * blockDim.x) {
        Run<S, V> in, out;
        load_bytes_stream<16>(xp + (size_t)r * V, &in);
        float f[V];
        decode_floats<DT, V>(in, f);
        #pragma unroll
        for (int j = 0; j < V; j++) f[j] = __double2float_rn(__dadd_rn(__dmul_rn((double)f[j], av), kv));
        encode_floats<DT, V>(f, out);
        store_bytes_stream<16>(yp + (size_t)r * V, &out);
    }
}

static bool pool_args(const char* name, const Tensor* X, Tensor* Y, const PoolParams* p) {
    if (!X || !Y || !p || !X->data || !Y->data || X->ndim != 4 || Y->ndim != 4 || !p->kernel_shape || !p->pads || !p->strides ||
        !p->dilations || Y->shape[0] != X->shape[0] || Y->shape[1] != X->shape[1] || p->strides[0] < 1 || p->strides[1] < 1 ||
        p->kernel_shape[0] < 1 || p->kernel_shape[1] < 1) {
        set_error(TOPS_ERR_INVALID, "%s: null argument, tensors that are not 4-D, or inconsistent shapes / attributes", name);
        zero_fill(Y);
        return false;
    }
    return true;
}

}  // namespace tops

using namespace tops;

TOPS_API void clip_forward(const Tensor* input, Tensor* output, const Tensor* min_t, const Tensor* max_t) {
    const char* name = "clip_forward";
    if (!input || !output || !input->data || !output->data || !dtype_valid((int)input->dtype) || !dtype_valid((int)output->dtype)) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor or bad dtype", name);
        zero_fill(output);
        return;
    }
    const bool has_lo = min_t && min_t->data, has_hi = max_t && max_t->data;
    const ShapeView out{output->shape, output->ndim, output->size};
    ShapeView ins[3] = {{input->shape, input->ndim, input->size}, {nullptr, 0, 1}, {nullptr, 0, 1}};
    const Tensor* bound[2] = {has_lo ? min_t : nullptr, has_hi ? max_t : nullptr};
    int n_ops = 1, where[2] = {-1, -1};
    for (int b = 0; b < 2; b++)
        if (bound[b]) { where[b] = n_ops; ins[n_ops++] = ShapeView{bound[b]->shape, bound[b]->ndim, bound[b]->size}; }
    Geometry geom;
    Operand ops[3];
    if (!plan_broadcast(out, ins, n_ops, &geom, ops)) {
        set_error(TOPS_ERR_INVALID, "%s: the bounds do not broadcast to the output's shape", name);
        zero_fill(output);
        return;
    }
    if (output->size == 0) return;
    if (output->size >= 0x7FFFFF00ull) { set_error(TOPS_ERR_UNSUPPORTED, "%s: more than 2^31 elements", name); return; }
    DeviceState* st = acquire_device();
    if (!st) return;
    ClipArgs a;
    a.g = geom;
    a.x = ops[0]; a.x.ptr = input->data; a.dx = (int)input->dtype;
    a.has_lo = has_lo; a.has_hi = has_hi;
    a.dlo = has_lo ? (int)min_t->dtype : DTYPE_FLOAT32;
    a.dhi = has_hi ? (int)max_t->dtype : DTYPE_FLOAT32;
    if (has_lo) { a.lo = ops[where[0]]; a.lo.ptr = min_t->data; }
    if (has_hi) { a.hi = ops[where[1]]; a.hi.ptr = max_t->data; }
    a.dout = (int)output->dtype;
    const int dt = (int)input->dtype;
    const bool scalar_bounds = (!has_lo || (min_t->size == 1 && dtype_exact_in_f32((int)min_t->dtype))) &&
                               (!has_hi || (max_t->size == 1 && dtype_exact_in_f32((int)max_t->dtype)));
    if (scalar_bounds && dt == (int)output->dtype && input->size == output->size && a.x.flat &&
        (((uintptr_t)input->data | (uintptr_t)output->data) & 15) == 0 &&
        (dt == DTYPE_FLOAT32 || dt == DTYPE_FLOAT16 || dt == DTYPE_BFLOAT16)) {
        const void* lo = has_lo ? min_t->data : nullptr;
        const void* hi = has_hi ? max_t->data : nullptr;
        const int grid = grid_for(output->size / 4 + 1, 256, st->sm_count, 8);
        if (dt == DTYPE_FLOAT32) clip_typed_kernel<DTYPE_FLOAT32><<<grid, 256, 0, current_stream()>>>(input->data, output->data, output->size, lo, a.dlo, hi, a.dhi);
        else if (dt == DTYPE_FLOAT16) clip_typed_kernel<DTYPE_FLOAT16><<<grid, 256, 0, current_stream()>>>(input->data, output->data, output->size, lo, a.dlo, hi, a.dhi);
        else clip_typed_kernel<DTYPE_BFLOAT16><<<grid, 256, 0, current_stream()>>>(input->data, output->data, output->size, lo, a.dlo, hi, a.dhi);
    } else {
        clip_kernel<<<grid_for(output->size, 256, st->sm_count, 8), 256, 0, current_stream()>>>(a, output->data, 0, (uint32_t)output->size);
    }
    TOPS_CHECK_LAUNCH(name);
    finish_op();
}

TOPS_API void average_pool_forward(const Tensor* X, Tensor* Y, PoolParams* params, int count_include_pad) {
    const char* name = "average_pool_forward";
    if (!pool_args(name, X, Y, params)) return;
    DeviceState* st = acquire_device();
    if (!st || Y->size == 0) return;
    AvgGeom p;
    p.C = X->shape[1]; p.H = X->shape[2]; p.W = X->shape[3]; p.OH = Y->shape[2]; p.OW = Y->shape[3];
    p.KH = params->kernel_shape[0]; p.KW = params->kernel_shape[1];
    p.pt = params->pads[0]; p.pl = params->pads[1];
    p.sh = params->strides[0]; p.sw = params->strides[1];
    p.dh = params->dilations[0]; p.dw = params->dilations[1];
    p.include_pad = count_include_pad ? 1 : 0;
    average_pool_kernel<<<grid_for(Y->size, 256, st->sm_count, 8), 256, 0, current_stream()>>>(X->data, Y->data, (int)X->dtype, (int)Y->dtype, p, Y->size);
    TOPS_CHECK_LAUNCH(name);
    finish_op();
}

TOPS_API void global_average_pool_forward(const Tensor* input, Tensor* output) {
    const char* name = "global_average_pool_forward";
    if (!input || !output || !input->data || !output->data || input->ndim != 4 ||
        output->size != (size_t)input->shape[0] * (size_t)input->shape[1]) {
        set_error(TOPS_ERR_INVALID, "%s: wants a 4-D input and one output element per plane", name);
        zero_fill(output);
        return;
    }
    DeviceState* st = acquire_device();
    if (!st || output->size == 0) return;
    const size_t planes = output->size;
    const int spatial = input->shape[2] * input->shape[3];
    const int dx = (int)input->dtype;
    if (dx == DTYPE_FLOAT32 || dx == DTYPE_FLOAT16 || dx == DTYPE_BFLOAT16) {
        const size_t groups = (planes + kGapPlanes - 1) / kGapPlanes;
        const int grid = grid_for(groups * 32, kGapWarps * 32, st->sm_count, 4);
        cudaStream_t s = current_stream();
        if (dx == DTYPE_FLOAT32) global_average_pool_typed<DTYPE_FLOAT32><<<grid, kGapWarps * 32, 0, s>>>(input->data, output->data, (int)output->dtype, planes, spatial);
        else if (dx == DTYPE_FLOAT16) global_average_pool_typed<DTYPE_FLOAT16><<<grid, kGapWarps * 32, 0, s>>>(input->data, output->data, (int)output->dtype, planes, spatial);
        else global_average_pool_typed<DTYPE_BFLOAT16><<<grid, kGapWarps * 32, 0, s>>>(input->data, output->data, (int)output->dtype, planes, spatial);
    } else {
        global_average_pool_kernel<<<grid_for(planes, 128, st->sm_count, 16), 128, 0, current_stream()>>>(input->data, output->data, dx,
                                                                                                     (int)output->dtype, planes, spatial);
    }
    TOPS_CHECK_LAUNCH(name);
    finish_op();
}

TOPS_API void batch_norm_forward(const Tensor* input, const Tensor* scale, const Tensor* B, const Tensor* mean, const Tensor* var,
                                 Tensor* output, float epsilon) {
    const char* name = "batch_norm_forward";
    if (!input || !scale || !B || !mean || !var || !output || !input->data || !output->data || input->ndim < 2 || input->size != output->size) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor, rank below 2 or size mismatch", name);
        zero_fill(output);
        return;
    }
    const int C = input->shape[1];
    const Tensor* tables[4] = {scale, B, mean, var};
    for (const Tensor* t : tables)
        if (!t->data || t->size < (size_t)C) { set_error(TOPS_ERR_INVALID, "%s: a per-channel operand is shorter than the channel count", name); zero_fill(output); return; }
    DeviceState* st = acquire_device();
    if (!st || output->size == 0) return;
    size_t spatial = 1;
    for (int d = 2; d < input->ndim; d++) spatial *= (size_t)input->shape[d];
    const size_t planes = (size_t)input->shape[0] * C;
    if (spatial >= 0x7FFFFFFFull || planes > 0x7FFFFFFFull) { set_error(TOPS_ERR_UNSUPPORTED, "%s: a dimension exceeds 2^31", name); return; }
    cudaStream_t s = current_stream();
    double* ak = nullptr;
    if (cudaMallocAsync((void**)&ak, sizeof(double) * 2 * (size_t)C, s) != cudaSuccess) { cudaGetLastError(); set_error(TOPS_ERR_OOM, "%s: scratch", name); return; }
    batch_norm_tables<<<(C + 127) / 128, 128, 0, s>>>(scale->data, B->data, mean->data, var->data, (int)scale->dtype, (int)B->dtype, (int)mean->dtype,
                                                      (int)var->dtype, (double)epsilon, C, ak, ak + C);
    // planes on grid.y (at most 65535 per launch), the plane's elements on grid.x
    const int dt = (int)input->dtype;
    const int vec = 16 / dtype_bytes(dt);
    const bool typed = dt == (int)output->dtype && (dt == DTYPE_FLOAT32 || dt == DTYPE_FLOAT16 || dt == DTYPE_BFLOAT16) && spatial % vec == 0 &&
                       (((uintptr_t)input->data | (uintptr_t)output->data) & 15) == 0;
    const size_t per_plane = typed ? spatial / vec : spatial;
    const unsigned gx = (unsigned)((per_plane + 255) / 256 < 64 ? (per_plane + 255) / 256 : 64);
    for (size_t first = 0; first < planes; first += 65535) {
        const unsigned gy = (unsigned)(planes - first < 65535 ? planes - first : 65535);
        const dim3 grid(gx ? gx : 1, gy);
        if (!typed) batch_norm_kernel<<<grid, 256, 0, s>>>(input->data, output->data, dt, (int)output->dtype, C, (uint32_t)spatial, ak, ak + C, first);
        else if (dt == DTYPE_FLOAT32) batch_norm_typed_kernel<DTYPE_FLOAT32><<<grid, 256, 0, s>>>(input->data, output->data, C, (uint32_t)spatial, ak, ak + C, first);
        else if (dt == DTYPE_FLOAT16) batch_norm_typed_kernel<DTYPE_FLOAT16><<<grid, 256, 0, s>>>(input->data, output->data, C, (uint32_t)spatial, ak, ak + C, first);
        else batch_norm_typed_kernel<DTYPE_BFLOAT16><<<grid, 256, 0, s>>>(input->data, output->data, C, (uint32_t)spatial, ak, ak + C, first);
    }
    TOPS_CHECK_LAUNCH(name);
    cudaFreeAsync(ak, s);
    finish_op();
}
