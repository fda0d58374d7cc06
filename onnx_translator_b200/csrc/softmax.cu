// Softmax along one axis (tensor_ops.c:1231-1270).  The tensor is viewed as [outer, inner, rem];
// each (outer, rem) pair is an independent row of `inner` elements with element stride `rem`.
//
//   rem == 1, inner <= 1024 : one warp per row, the row lives in registers, max and sum by
//                             warp shuffles.
//   rem == 1, inner  > 1024 : one CTA per row, the decoded row staged in shared memory.
//   rem  > 1 (or any other) : one thread per row walking it with stride `rem` (neighbouring
//                             threads touch neighbouring addresses), in the reference's own
//                             sequential order.
// Arithmetic is double throughout, as in the reference; the differences are the order of the
// additions in the parallel sums, a leaner exp (1e-11 relative) and multiplication by 1 / sum
// instead of a division per element: results agree to the last float32 bit or one ulp.
#include "common.cuh"
#include "elementwise.cuh"
#include "umma.cuh"

#include <cfloat>

namespace tops {

template <int DT> __device__ __forceinline__ double sm_load(const void* p, int rt, size_t i) {
    if constexpr (DT < 0) return load_f64_rt(p, rt, i);
    else return to_f64<DT>(((const typename Storage<DT>::type*)p)[i]);
}
template <int DT> __device__ __forceinline__ void sm_store(void* p, int rt, size_t i, double v) {
    if constexpr (DT < 0) store_f64_rt(p, rt, i, v);
    else ((typename Storage<DT>::type*)p)[i] = from_f64<DT>(v);
}

__device__ __forceinline__ double warp_max(double v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// exp(d) for d <= 0 (every softmax argument is value - max) in double, accurate to about 1e-11
// relative -- far inside the float32 rounding of the result and the 1e-6 gate of the tests, and
// less than half the fp64 instructions of the general-purpose exp: k = rint(d / ln 2) by a magic
// add, r = d - k ln 2 with a two-part ln 2, a degree-9 Taylor polynomial (|r| <= 0.347), and the
// scaling by 2^k done on the exponent bits.  Results below 2^-1021 are flushed to zero (they are
// below 1e-307 of the largest term); NaN stays NaN.
__device__ __forceinline__ double exp_nonpositive(double d) {
    if (!(d >= -707.0)) return d != d ? d : 0.0;
    const double kMagic = 6755399441055744.0;                       // 1.5 * 2^52
    const double t = fma(d, 1.4426950408889634, kMagic);
    const int k = __double2loint(t);
    const double kf = t - kMagic;
    double r = fma(kf, -6.93147180369123816490e-01, d);             // ln 2, high part
    r = fma(kf, -1.90821492927058770002e-10, r);                    // ln 2, low part
    double p = 2.7557319223985893e-06;                              // 1/9!
    p = fma(p, r, 2.48015873015873e-05);
    p = fma(p, r, 1.984126984126984e-04);
    p = fma(p, r, 1.388888888888889e-03);
    p = fma(p, r, 8.333333333333333e-03);
    p = fma(p, r, 4.1666666666666664e-02);
    p = fma(p, r, 1.6666666666666666e-01);
    p = fma(p, r, 0.5);
    p = fma(p, r, 1.0);
    p = fma(p, r, 1.0);
    return __hiloint2double(__double2hiint(p) + (k << 20), __double2loint(p));
}

// NaN handling follows the strict '>' scan of the reference: NaN never becomes the maximum.
__device__ __forceinline__ double max_step(double best, double v) { return v > best ? v : best; }

constexpr int kWarpRowMax = 1024;
constexpr int kWarpRowPerLane = kWarpRowMax / 32;

// One warp per row, any dtype pair: the row lives in double registers, arithmetic as the reference.
template <int DX, int DO>
__global__ void __launch_bounds__(256) softmax_warp_rows(const void* __restrict__ x, void* __restrict__ y,
                                                          int dx, int dout, uint32_t rows, uint32_t inner) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps_per_grid) {
        const size_t base = (size_t)row * inner;
        {
            double v[kWarpRowPerLane];
            double top = -DBL_MAX;
            #pragma unroll
            for (int k = 0; k < kWarpRowPerLane; k++) {
                const uint32_t j = lane + 32u * k;
                if (j < inner) { v[k] = sm_load<DX>(x, dx, base + j); top = max_step(top, v[k]); }
            }
            #pragma unroll
            for (int o = 16; o > 0; o >>= 1) top = max_step(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
            double total = 0.0;
            #pragma unroll
            for (int k = 0; k < kWarpRowPerLane; k++) {
                const uint32_t j = lane + 32u * k;
                if (j < inner) { v[k] = exp_nonpositive(v[k] - top); total += v[k]; }
            }
            total = warp_sum(total);
            const double inv = 1.0 / total;
            #pragma unroll
            for (int k = 0; k < kWarpRowPerLane; k++) {
                const uint32_t j = lane + 32u * k;
                if (j < inner) sm_store<DO>(y, dout, base + j, v[k] * inv);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// float32 / float16 / bfloat16 rows of up to 1024 elements: one warp per row, rows staged in shared
// memory.  Each warp owns two row buffers; while it works on one row, the next row is already being
// copied into the other buffer by an untiled bulk copy (cp.async.bulk) that signals an mbarrier, so
// the memory system always has a row per warp in flight and the arithmetic never waits for a load it
// has just issued.  Rows whose start or length is not a multiple of 16 bytes are staged by plain
// coalesced loads instead (BULK = false).
//
// The arithmetic is float32 with two compensations and stays within 5e-7 relative of the reference's
// double evaluation (gate of the tests: 1e-6); results below the normal range of the output type may
// differ by one denormal step, since the exponential itself is then a rounded denormal:
//   * value - max is formed as a two-float sum (TwoSum), exp(hi + lo) = exp(hi) * (1 + lo);
//   * exp is the accurate expf (2 ulp); four terms are added pairwise in float, the groups in double;
//   * normalisation is one multiplication by the correctly rounded 1 / sum.
// About 25 instructions per element instead of about 100 for the all-double formulation.
// ---------------------------------------------------------------------------------------------
using namespace umma;
constexpr int kStagedWarps = 4;

template <int DT> __device__ __forceinline__ void staged_load4(const unsigned char* row, uint32_t g, float (&f)[4]) {
    if constexpr (dtype_bytes(DT) == 4) {
        const float4 v = *reinterpret_cast<const float4*>(row + 16u * g);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    } else {
        const uint2 v = *reinterpret_cast<const uint2*>(row + 8u * g);
        if constexpr (DT == DTYPE_FLOAT16) {
            const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x));
            const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
            f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y;
        } else {                                                   // bfloat16: the upper half of a float32
            f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
            f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
        }
    }
}

template <int DT> __device__ __forceinline__ typename Storage<DT>::type minus_inf_stored() {
    if constexpr (DT == DTYPE_FLOAT32) return __uint_as_float(0xFF800000u);
    else return (typename Storage<DT>::type)(DT == DTYPE_FLOAT16 ? 0xFC00u : 0xFF80u);
}

template <int DT, bool BULK, bool VEC_OUT>
__global__ void __launch_bounds__(kStagedWarps * 32) softmax_rows_staged(const typename Storage<DT>::type* __restrict__ x,
                                                                          typename Storage<DT>::type* __restrict__ y,
                                                                          uint32_t rows, uint32_t inner, int* status) {
    using S = typename Storage<DT>::type;
    constexpr uint32_t ES = sizeof(S);
    extern __shared__ __align__(128) unsigned char staged_smem[];
    __shared__ int abort_flag;
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    const uint32_t groups = (inner + 3u) >> 2;                       // groups of four elements
    const uint32_t row_pad = (groups * 4u * ES + 15u) & ~15u;         // bytes of one staging buffer
    const uint32_t e_bytes = ES == 4 ? 0u : groups * 16u;             // 4-byte rows hold exp() in place
    uint64_t* bars = reinterpret_cast<uint64_t*>(staged_smem) + 2u * warp;
    unsigned char* mine = staged_smem + 16u * kStagedWarps + warp * (2u * row_pad + e_bytes);
    if (threadIdx.x == 0) abort_flag = 0;
    if (BULK && lane == 0) { mbar_init(&bars[0], 1); mbar_init(&bars[1], 1); mbar_fence_init(); }
    __syncthreads();

    const uint32_t stride = gridDim.x * kStagedWarps;
    uint32_t row = blockIdx.x * kStagedWarps + warp;
    const uint32_t row_bytes = inner * ES;
    if (BULK && row < rows && lane == 0) {
        mbar_expect_tx(&bars[0], row_bytes);
        bulk_load_1d(mine, x + (size_t)row * inner, row_bytes, &bars[0]);
    }
    uint32_t phases = 0;
    for (uint32_t buf = 0; row < rows; row += stride, buf ^= 1u) {
        unsigned char* cur = mine + buf * row_pad;
        if constexpr (BULK) {
            const uint32_t next = row + stride;
            if (next < rows) {
                // the other buffer was read and written by this warp one iteration ago
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    mbar_expect_tx(&bars[buf ^ 1u], row_bytes);
                    bulk_load_1d(mine + (buf ^ 1u) * row_pad, x + (size_t)next * inner, row_bytes, &bars[buf ^ 1u]);
                }
            }
            if (!mbar_wait(&bars[buf], (phases >> buf) & 1u, &abort_flag)) break;
            phases ^= 1u << buf;
        } else {
            __syncwarp();
            const S* src = x + (size_t)row * inner;
            for (uint32_t j = lane; j < groups * 4u; j += 32u)
                reinterpret_cast<S*>(cur)[j] = j < inner ? src[j] : minus_inf_stored<DT>();
            __syncwarp();
        }
        float* ebuf = ES == 4 ? reinterpret_cast<float*>(cur) : reinterpret_cast<float*>(mine + 2u * row_pad);

        float top = -FLT_MAX;                      // stands in for the reference's -DBL_MAX start value
        for (uint32_t g = lane; g < groups; g += 32u) {
            float f[4];
            staged_load4<DT>(cur, g, f);
            #pragma unroll
            for (int q = 0; q < 4; q++) top = f[q] > top ? f[q] : top;   // strict '>': NaN is never the maximum
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) { const float t = __shfl_xor_sync(0xFFFFFFFFu, top, o); top = t > top ? t : top; }

        double total = 0.0;
        for (uint32_t g = lane; g < groups; g += 32u) {
            float f[4];
            staged_load4<DT>(cur, g, f);
            #pragma unroll
            for (int q = 0; q < 4; q++) {
                // two-float difference: hi + lo == value - top exactly (when finite)
                const float hi = __fsub_rn(f[q], top);
                const float bb = __fsub_rn(hi, f[q]);
                const float lo = __fadd_rn(__fsub_rn(f[q], __fsub_rn(hi, bb)), __fsub_rn(-top, bb));
                float e = expf(hi);
                if (lo == lo && e > 0.0f) e = fmaf(e, lo, e);
                f[q] = e;
            }
            *reinterpret_cast<float4*>(ebuf + 4u * g) = make_float4(f[0], f[1], f[2], f[3]);
            total += (double)__fadd_rn(__fadd_rn(f[0], f[1]), __fadd_rn(f[2], f[3]));
        }
        total = warp_sum(total);
        const float inv = __double2float_rn(1.0 / total);

        S* dst = y + (size_t)row * inner;
        for (uint32_t g = lane; g < groups; g += 32u) {
            const float4 e = *reinterpret_cast<const float4*>(ebuf + 4u * g);
            const float r[4] = {__fmul_rn(e.x, inv), __fmul_rn(e.y, inv), __fmul_rn(e.z, inv), __fmul_rn(e.w, inv)};
            if constexpr (VEC_OUT) {
                if constexpr (ES == 4) {
                    *reinterpret_cast<float4*>(dst + 4u * g) = make_float4(r[0], r[1], r[2], r[3]);
                } else {
                    uint2 packed;
                    packed.x = DT == DTYPE_FLOAT16 ? encode_f16x2(r[0], r[1]) : encode_bf16x2(r[0], r[1]);
                    packed.y = DT == DTYPE_FLOAT16 ? encode_f16x2(r[2], r[3]) : encode_bf16x2(r[2], r[3]);
                    *reinterpret_cast<uint2*>(dst + 4u * g) = packed;
                }
            } else {
                #pragma unroll
                for (int q = 0; q < 4; q++) if (4u * g + q < inner) dst[4u * g + q] = from_f32<DT>(r[q]);
            }
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 1);
}

template <int DT>
static void softmax_staged_launch(const Tensor* x, Tensor* y, uint32_t rows, uint32_t inner, DeviceState* st, cudaStream_t s) {
    using S = typename Storage<DT>::type;
    constexpr uint32_t ES = sizeof(S);
    const uint32_t groups = (inner + 3u) >> 2;
    const uint32_t row_pad = (groups * 4u * ES + 15u) & ~15u;
    const size_t smem = 16u * kStagedWarps + (size_t)kStagedWarps * (2u * row_pad + (ES == 4 ? 0u : groups * 16u));
    const bool bulk = ((size_t)inner * ES) % 16 == 0 && ((uintptr_t)x->data % 16) == 0;
    const bool vec_out = inner % 4 == 0 && ((uintptr_t)y->data % (4 * ES)) == 0;
    size_t ctas_per_sm = (size_t)(220 * 1024) / (smem + 1024);
    if (ctas_per_sm > 12) ctas_per_sm = 12;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    const size_t want = ((size_t)rows + kStagedWarps - 1) / kStagedWarps;
    const size_t cap = (size_t)st->sm_count * ctas_per_sm;
    const int grid = (int)(want < cap ? want : cap);
    const S* xp = (const S*)x->data;
    S* yp = (S*)y->data;
    int* status = bulk ? device_status_word() : nullptr;
#define TOPS_STAGED(B, V) softmax_rows_staged<DT, B, V><<<grid, kStagedWarps * 32, smem, s>>>(xp, yp, rows, inner, status)
    if (bulk) { if (vec_out) TOPS_STAGED(true, true); else TOPS_STAGED(true, false); }
    else      { if (vec_out) TOPS_STAGED(false, true); else TOPS_STAGED(false, false); }
#undef TOPS_STAGED
}

template <int DX, int DO>
__global__ void __launch_bounds__(512) softmax_block_rows(const void* __restrict__ x, void* __restrict__ y,
                                                           int dx, int dout, uint32_t rows, uint32_t inner, int staged) {
    extern __shared__ double row_buf[];
    __shared__ double red[16];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * inner;
        double top = -DBL_MAX;
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double v = sm_load<DX>(x, dx, base + j);
            if (staged) row_buf[j] = v;
            top = max_step(top, v);
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = max_step(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
        if (lane == 0) red[warp] = top;
        __syncthreads();
        top = -DBL_MAX;
        for (uint32_t w = 0; w < nwarps; w++) top = max_step(top, red[w]);
        __syncthreads();
        double total = 0.0;
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double e = exp_nonpositive((staged ? row_buf[j] : sm_load<DX>(x, dx, base + j)) - top);
            if (staged) row_buf[j] = e;
            total += e;
        }
        total = warp_sum(total);
        if (lane == 0) red[warp] = total;
        __syncthreads();
        total = 0.0;
        for (uint32_t w = 0; w < nwarps; w++) total += red[w];
        const double inv = 1.0 / total;
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double e = staged ? row_buf[j] : exp_nonpositive(sm_load<DX>(x, dx, base + j) - top);
            sm_store<DO>(y, dout, base + j, e * inv);
        }
        __syncthreads();
    }
}

template <int DX, int DO>
__global__ void __launch_bounds__(256) softmax_strided_rows(const void* __restrict__ x, void* __restrict__ y,
                                                             int dx, int dout, uint32_t outer, uint32_t inner, uint32_t rem) {
    const size_t rows = (size_t)outer * rem;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (size_t)gridDim.x * blockDim.x) {
        const size_t o = r / rem, k = r - o * rem;
        const size_t base = o * inner * rem + k;
        double top = -DBL_MAX;
        for (uint32_t j = 0; j < inner; j++) top = max_step(top, sm_load<DX>(x, dx, base + (size_t)j * rem));
        double total = 0.0;
        for (uint32_t j = 0; j < inner; j++) total += exp_nonpositive(sm_load<DX>(x, dx, base + (size_t)j * rem) - top);
        const double inv = 1.0 / total;
        for (uint32_t j = 0; j < inner; j++) {
            const size_t idx = base + (size_t)j * rem;
            sm_store<DO>(y, dout, idx, exp_nonpositive(sm_load<DX>(x, dx, idx) - top) * inv);
        }
    }
}

template <int DX, int DO>
static void softmax_launch(const Tensor* x, Tensor* y, uint32_t outer, uint32_t inner, uint32_t rem, DeviceState* st) {
    cudaStream_t s = current_stream();
    const int dx = (int)x->dtype, dout = (int)y->dtype;
    if constexpr (DX >= 0 && DX == DO) {
        if (rem == 1 && inner <= kWarpRowMax && inner >= 16) {
            softmax_staged_launch<(DX >= 0 ? DX : DTYPE_FLOAT32)>(x, y, outer, inner, st, s);
            TOPS_CHECK_LAUNCH("softmax_forward");
            return;
        }
    }
    if (rem == 1 && inner <= kWarpRowMax && inner >= 16) {
        const int grid = grid_for((size_t)outer * 32, 256, st->sm_count, 8);
        softmax_warp_rows<DX, DO><<<grid, 256, 0, s>>>(x->data, y->data, dx, dout, outer, inner);
    } else if (rem == 1 && inner > kWarpRowMax) {
        const size_t need = (size_t)inner * sizeof(double);
        const int staged = need <= 200 * 1024;
        if (staged) cudaFuncSetAttribute(softmax_block_rows<DX, DO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        const int grid = (int)((outer < (uint32_t)st->sm_count * 2) ? outer : (uint32_t)st->sm_count * 2);
        softmax_block_rows<DX, DO><<<grid, 512, staged ? need : 0, s>>>(x->data, y->data, dx, dout, outer, inner, staged);
    } else {
        const int grid = grid_for((size_t)outer * rem, 256, st->sm_count, 8);
        softmax_strided_rows<DX, DO><<<grid, 256, 0, s>>>(x->data, y->data, dx, dout, outer, inner, rem);
    }
    TOPS_CHECK_LAUNCH("softmax_forward");
}

}  // namespace tops

using namespace tops;

TOPS_API void softmax_forward(const Tensor* input, Tensor* output, int axis) {
    if (!input || !output || !input->data || !output->data || input->size != output->size || input->ndim < 1) {
        set_error(TOPS_ERR_INVALID, "softmax_forward: null tensor, size mismatch or rank 0");
        zero_fill(output);
        return;
    }
    if (axis < 0) axis += input->ndim;
    if (axis < 0 || axis >= input->ndim) { set_error(TOPS_ERR_INVALID, "softmax_forward: axis out of range"); zero_fill(output); return; }
    DeviceState* st = acquire_device();
    if (!st || input->size == 0) return;
    size_t outer = 1, rem = 1;
    const size_t inner = (size_t)input->shape[axis];
    for (int d = 0; d < axis; d++) outer *= (size_t)input->shape[d];
    for (int d = axis + 1; d < input->ndim; d++) rem *= (size_t)input->shape[d];
    if (outer > 0x7FFFFFFFull || inner > 0x7FFFFFFFull || rem > 0x7FFFFFFFull) {
        set_error(TOPS_ERR_UNSUPPORTED, "softmax_forward: a dimension exceeds 2^31");
        return;
    }
    const int dx = (int)input->dtype, dout = (int)output->dtype;
    if (dx == DTYPE_FLOAT32 && dout == DTYPE_FLOAT32)        softmax_launch<DTYPE_FLOAT32, DTYPE_FLOAT32>(input, output, outer, inner, rem, st);
    else if (dx == DTYPE_FLOAT16 && dout == DTYPE_FLOAT16)   softmax_launch<DTYPE_FLOAT16, DTYPE_FLOAT16>(input, output, outer, inner, rem, st);
    else if (dx == DTYPE_BFLOAT16 && dout == DTYPE_BFLOAT16) softmax_launch<DTYPE_BFLOAT16, DTYPE_BFLOAT16>(input, output, outer, inner, rem, st);
    else                                                     softmax_launch<-1, -1>(input, output, outer, inner, rem, st);
    finish_op();
}
