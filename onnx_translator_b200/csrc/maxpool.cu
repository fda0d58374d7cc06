// MaxPool over NCHW planes (tensor_ops.c:1116-1165): scan the window kh -> kw from -Inf with a
// strict '>', skip taps outside the plane.  NaN is therefore never selected and a window made
// only of padding yields -Inf.  Selection is exact, so the output is bit-identical by construction.
//
// One thread per output element, neighbouring threads along the output row: loads of a warp are
// contiguous (stride-1 pools) or stride-s segments of the same input rows, and the kh/kw re-reads
// of overlapping windows are served by L1.  max_pool_kernel is the general form (any dtype pair,
// 64-bit indices); max_pool_win below is the fast form for same-dtype pools.
#include "common.cuh"

namespace tops {

struct PoolGeom {
    int C, H, W, OH, OW, KH, KW, pt, pl, sh, sw, dh, dw;
};

template <int DX, int DO>
__global__ void __launch_bounds__(256) max_pool_kernel(const void* __restrict__ x, void* __restrict__ y,
                                                        int dx, int dout, PoolGeom p, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ow = (int)(i % (size_t)p.OW);
        const size_t t = i / (size_t)p.OW;
        const int oh = (int)(t % (size_t)p.OH);
        const size_t plane = t / (size_t)p.OH;                    // n * C + c
        const size_t in_base = plane * (size_t)p.H * (size_t)p.W;
        const int h0 = oh * p.sh - p.pt, w0 = ow * p.sw - p.pl;
        if constexpr (DX >= 0 && dtype_exact_in_f32(DX >= 0 ? DX : 0)) {
            using S = typename Storage<(DX >= 0 ? DX : 0)>::type;
            const S* src = (const S*)x + in_base;
            float best = -INFINITY;
            for (int kh = 0; kh < p.KH; kh++) {
                const int ih = h0 + kh * p.dh;
                if (ih < 0 || ih >= p.H) continue;
                for (int kw = 0; kw < p.KW; kw++) {
                    const int iw = w0 + kw * p.dw;
                    if (iw < 0 || iw >= p.W) continue;
                    const float v = to_f32<(DX >= 0 ? DX : 0)>(src[(size_t)ih * p.W + iw]);
                    if (v > best) best = v;
                }
            }
            if constexpr (dtype_is_int(DO >= 0 ? DO : 0))
                ((typename Storage<(DO >= 0 ? DO : 0)>::type*)y)[i] = from_f64<(DO >= 0 ? DO : 0)>((double)best);
            else
                ((typename Storage<(DO >= 0 ? DO : 0)>::type*)y)[i] = from_f32<(DO >= 0 ? DO : 0)>(best);
        } else {
            double best = -INFINITY;
            for (int kh = 0; kh < p.KH; kh++) {
                const int ih = h0 + kh * p.dh;
                if (ih < 0 || ih >= p.H) continue;
                for (int kw = 0; kw < p.KW; kw++) {
                    const int iw = w0 + kw * p.dw;
                    if (iw < 0 || iw >= p.W) continue;
                    const double v = load_f64_rt(x, dx, in_base + (size_t)ih * p.W + iw);
                    if (v > best) best = v;
                }
            }
            store_f64_rt(y, dout, i, best);
        }
    }
}

// Same-dtype kernel for the dtypes whose values are exact in float32.  The window extents are
// template parameters for the usual 2x2 and 3x3 pools (the tap loops unroll and the loads of one
// window are all in flight together) and run-time values otherwise (KH == 0); the output index is
// 32-bit and is taken apart with multiply-high divisions, so one output costs a few dozen
// instructions instead of the several hundred of the 64-bit generic kernel.
template <int DT, int KH, int KW>
__global__ void __launch_bounds__(256) max_pool_win(const typename Storage<DT>::type* __restrict__ x,
                                                     typename Storage<DT>::type* __restrict__ y, PoolGeom p,
                                                     FastDiv by_ow, FastDiv by_oh, uint32_t total) {
    const int kh_n = KH ? KH : p.KH, kw_n = KW ? KW : p.KW;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const uint32_t t = by_ow.div(i), ow = i - t * (uint32_t)p.OW;
        const uint32_t plane = by_oh.div(t), oh = t - plane * (uint32_t)p.OH;
        const typename Storage<DT>::type* src = x + (size_t)plane * (size_t)(p.H * p.W);
        const int h0 = (int)oh * p.sh - p.pt, w0 = (int)ow * p.sw - p.pl;
        float best = -INFINITY;
        #pragma unroll
        for (int kh = 0; kh < kh_n; kh++) {
            const int ih = h0 + kh * p.dh;
            if ((unsigned)ih >= (unsigned)p.H) continue;
            const typename Storage<DT>::type* row = src + ih * p.W;
            #pragma unroll
            for (int kw = 0; kw < kw_n; kw++) {
                const int iw = w0 + kw * p.dw;
                if ((unsigned)iw >= (unsigned)p.W) continue;
                const float v = to_f32<DT>(row[iw]);
                if (v > best) best = v;
            }
        }
        if constexpr (dtype_is_int(DT)) y[i] = from_f64<DT>((double)best);
        else y[i] = from_f32<DT>(best);
    }
}

template <int DT>
static void launch_win(const Tensor* X, Tensor* Y, const PoolGeom& p, DeviceState* st, cudaStream_t s) {
    using S = typename Storage<DT>::type;
    FastDiv by_ow, by_oh;
    by_ow.set((uint32_t)p.OW);
    by_oh.set((uint32_t)p.OH);
    const uint32_t total = (uint32_t)Y->size;
    const int grid = grid_for(Y->size, 256, st->sm_count, 8);
    const S* x = (const S*)X->data;
    S* y = (S*)Y->data;
    if (p.KH == 2 && p.KW == 2)      max_pool_win<DT, 2, 2><<<grid, 256, 0, s>>>(x, y, p, by_ow, by_oh, total);
    else if (p.KH == 3 && p.KW == 3) max_pool_win<DT, 3, 3><<<grid, 256, 0, s>>>(x, y, p, by_ow, by_oh, total);
    else                             max_pool_win<DT, 0, 0><<<grid, 256, 0, s>>>(x, y, p, by_ow, by_oh, total);
}

}  // namespace tops

using namespace tops;

TOPS_API void max_pool_forward(const Tensor* X, Tensor* Y, PoolParams* params) {
    if (!X || !Y || !params || !X->data || !Y->data || X->ndim != 4 || Y->ndim != 4 ||
        !params->kernel_shape || !params->pads || !params->strides || !params->dilations) {
        set_error(TOPS_ERR_INVALID, "max_pool_forward: null argument or tensors that are not 4-D");
        zero_fill(Y);
        return;
    }
    PoolGeom p;
    p.C = X->shape[1]; p.H = X->shape[2]; p.W = X->shape[3];
    p.OH = Y->shape[2]; p.OW = Y->shape[3];
    p.KH = params->kernel_shape[0]; p.KW = params->kernel_shape[1];
    p.pt = params->pads[0]; p.pl = params->pads[1];
    p.sh = params->strides[0]; p.sw = params->strides[1];
    p.dh = params->dilations[0]; p.dw = params->dilations[1];
    if (Y->shape[0] != X->shape[0] || Y->shape[1] != X->shape[1] || p.sh < 1 || p.sw < 1 || p.KH < 1 || p.KW < 1) {
        set_error(TOPS_ERR_INVALID, "max_pool_forward: inconsistent shapes or attributes");
        zero_fill(Y);
        return;
    }
    DeviceState* st = acquire_device();
    if (!st || Y->size == 0) return;
    const int grid = grid_for(Y->size, 256, st->sm_count, 8);
    cudaStream_t s = current_stream();
    const int dx = (int)X->dtype, dout = (int)Y->dtype;
    // 32-bit indexing: outputs, one input plane and the span of a window all below 2^31
    if (dx == dout && Y->size < 0x7FFFFFFFull && (size_t)p.H * p.W < 0x7FFFFFFFull &&
        (size_t)p.OH * p.sh + (size_t)p.KH * p.dh < 0x7FFFFFFFull && (size_t)p.OW * p.sw + (size_t)p.KW * p.dw < 0x7FFFFFFFull) {
        bool launched = true;
        switch (dx) {
            case DTYPE_FLOAT32:     launch_win<DTYPE_FLOAT32>(X, Y, p, st, s); break;
            case DTYPE_FLOAT16:     launch_win<DTYPE_FLOAT16>(X, Y, p, st, s); break;
            case DTYPE_BFLOAT16:    launch_win<DTYPE_BFLOAT16>(X, Y, p, st, s); break;
            case DTYPE_INT8:        launch_win<DTYPE_INT8>(X, Y, p, st, s); break;
            case DTYPE_UINT8:       launch_win<DTYPE_UINT8>(X, Y, p, st, s); break;
            case DTYPE_FLOAT8_E4M3: launch_win<DTYPE_FLOAT8_E4M3>(X, Y, p, st, s); break;
            case DTYPE_FLOAT8_E5M2: launch_win<DTYPE_FLOAT8_E5M2>(X, Y, p, st, s); break;
            default: launched = false;
        }
        if (launched) {
            TOPS_CHECK_LAUNCH("max_pool_forward");
            finish_op();
            return;
        }
    }
#define TOPS_POOL(T) if (dx == T && dout == T) { max_pool_kernel<T, T><<<grid, 256, 0, s>>>(X->data, Y->data, dx, dout, p, Y->size); } else
    TOPS_POOL(DTYPE_FLOAT32) TOPS_POOL(DTYPE_FLOAT16) TOPS_POOL(DTYPE_BFLOAT16) TOPS_POOL(DTYPE_INT8)
    TOPS_POOL(DTYPE_UINT8) TOPS_POOL(DTYPE_FLOAT8_E4M3) TOPS_POOL(DTYPE_FLOAT8_E5M2)
    { max_pool_kernel<-1, -1><<<grid, 256, 0, s>>>(X->data, Y->data, dx, dout, p, Y->size); }
#undef TOPS_POOL
    TOPS_CHECK_LAUNCH("max_pool_forward");
    finish_op();
}
