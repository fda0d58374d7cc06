// MaxPool over NCHW planes (tensor_ops.c:1116-1165): scan the window kh -> kw from -Inf with a
// strict '>', skip taps outside the plane.  NaN is therefore never selected and a window made
// only of padding yields -Inf.  Selection is exact, so the output is bit-identical by construction.
//
// One thread per output element, neighbouring threads along the output row: loads of a warp are
// contiguous (stride-1 pools) or stride-s segments of the same input rows, and the kh/kw re-reads
// of overlapping windows are served by L1.  max_pool_kernel is the general form (any dtype pair,
// 64-bit indices); max_pool_win below is the fast form for same-dtype pools.
#include "elementwise.cuh"

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

template <int DT> static bool launch_stride2(const Tensor* X, Tensor* Y, const PoolGeom& p, DeviceState* st, cudaStream_t s);

template <int DT>
static void launch_win(const Tensor* X, Tensor* Y, const PoolGeom& p, DeviceState* st, cudaStream_t s) {
    using S = typename Storage<DT>::type;
    if (launch_stride2<DT>(X, Y, p, st, s)) return;
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

// ---------------------------------------------------------------------------------------------
// The two stride-2 pools of convolutional networks -- 2x2 without padding and 3x3 with one cell of
// padding -- on planes whose width is a multiple of four.  A thread owns four input columns (one
// 16-byte load for float32), hence two output columns, and walks down a strip of output rows:
// every input row is loaded once, reduced along the row first (the left neighbour of the 3x3
// window comes from the neighbouring lane by a shuffle), then combined down the column, with the
// row shared by two vertically adjacent 3x3 windows carried in registers.  The tap order of the
// reference (row by row, left to right, strict '>') is kept, so ties between +0 and -0 and the
// NaN rule resolve identically.
// ---------------------------------------------------------------------------------------------
template <int DT> __device__ __forceinline__ void pool_load4(const typename Storage<DT>::type* p, bool on, float (&v)[4]) {
    using S = typename Storage<DT>::type;
    v[0] = v[1] = v[2] = v[3] = -INFINITY;
    if (!on) return;
    S raw[4];
    load_bytes<4 * (int)sizeof(S)>(p, raw);
    #pragma unroll
    for (int j = 0; j < 4; j++) v[j] = to_f32<DT>(raw[j]);
}

template <int DT, int K, int STRIP>
__global__ void __launch_bounds__(256) max_pool_stride2_strips(const typename Storage<DT>::type* __restrict__ x,
                                                                typename Storage<DT>::type* __restrict__ y,
                                                                int H, int W, int OH, int OW, uint32_t quads,
                                                                uint32_t strips, FastDiv by_quads, FastDiv by_strips, uint32_t total) {
    using S = typename Storage<DT>::type;
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x, lane = threadIdx.x & 31u;
    const bool live = i < total;
    const uint32_t t = by_quads.div(i), q = i - t * quads;
    const uint32_t plane = by_strips.div(t), part = t - plane * strips;
    const int oh0 = (int)part * STRIP;
    const S* src = x + (size_t)plane * (size_t)(H * W) + 4u * q;
    S* dst = y + (size_t)plane * (size_t)(OH * OW) + 2u * q;

    // Phase 1: every input row of the strip is requested before any is used (2 * STRIP rows, plus the row above for the
    // 3x3 pool), so a thread has all of its loads in flight at once.
    constexpr int kRows = 2 * STRIP + (K == 3 ? 1 : 0);
    const int first_row = 2 * oh0 - (K == 3 ? 1 : 0);
    float v[kRows][4];
    float left_edge[kRows];                                           // column 4q - 1 for lane 0 of a warp that starts inside a row
    bool on[kRows];
    #pragma unroll
    for (int r = 0; r < kRows; r++) {
        const int ih = first_row + r;
        // the row above the strip exists for every strip but the first; rows 2 * oh and 2 * oh + 1 exist when output row oh does
        const int rr = K == 3 ? (r - 1) >> 1 : r >> 1;
        on[r] = (K == 3 && r == 0) ? (live && oh0 > 0 && oh0 < OH) : (live && oh0 + rr < OH);
        pool_load4<DT>(src + ih * W, on[r], v[r]);
        left_edge[r] = -INFINITY;
        if constexpr (K == 3) if (lane == 0 && q != 0 && on[r]) left_edge[r] = to_f32<DT>(src[ih * W - 1]);
    }
    // Phase 2: horizontal maxima of each row for this thread's two output columns, then down the columns.  The tap
    // order of the reference (row by row, left to right, strict '>') is kept.
    auto row_maxima = [&](int r, float& m0, float& m1) {
        m0 = -INFINITY; m1 = -INFINITY;
        if constexpr (K == 3) {
            float left = __shfl_up_sync(0xFFFFFFFFu, v[r][3], 1);     // column 4q - 1 lives in the lane to the left
            if (q == 0) left = -INFINITY;                             // padding column
            else if (lane == 0) left = left_edge[r];
            if (left > m0) m0 = left;
            if (v[r][0] > m0) m0 = v[r][0];
            if (v[r][1] > m0) m0 = v[r][1];
            if (v[r][1] > m1) m1 = v[r][1];
            if (v[r][2] > m1) m1 = v[r][2];
            if (v[r][3] > m1) m1 = v[r][3];
        } else {
            if (v[r][0] > m0) m0 = v[r][0];
            if (v[r][1] > m0) m0 = v[r][1];
            if (v[r][2] > m1) m1 = v[r][2];
            if (v[r][3] > m1) m1 = v[r][3];
        }
    };
    float carry0 = -INFINITY, carry1 = -INFINITY;                     // the row above the strip (3x3 only)
    if constexpr (K == 3) row_maxima(0, carry0, carry1);
    #pragma unroll
    for (int r = 0; r < STRIP; r++) {
        const int oh = oh0 + r;
        const bool row_on = live && oh < OH;
        float a0, a1, b0, b1;
        row_maxima(2 * r + (K == 3 ? 1 : 0), a0, a1);
        row_maxima(2 * r + 1 + (K == 3 ? 1 : 0), b0, b1);
        float o0 = carry0, o1 = carry1;                               // -Inf for the 2x2 pool
        if (a0 > o0) o0 = a0;
        if (a1 > o1) o1 = a1;
        if (b0 > o0) o0 = b0;
        if (b1 > o1) o1 = b1;
        if constexpr (K == 3) { carry0 = b0; carry1 = b1; }
        if (row_on) {
            S out[2];
            if constexpr (dtype_is_int(DT)) { out[0] = from_f64<DT>((double)o0); out[1] = from_f64<DT>((double)o1); }
            else { out[0] = from_f32<DT>(o0); out[1] = from_f32<DT>(o1); }
            store_bytes_stream<2 * (int)sizeof(S)>(dst + oh * OW, out);
        }
    }
}

// false: the shape is not one of the two stride-2 pools this kernel covers
template <int DT>
static bool launch_stride2(const Tensor* X, Tensor* Y, const PoolGeom& p, DeviceState* st, cudaStream_t s) {
    using S = typename Storage<DT>::type;
    const int K = p.KH;
    if (!(p.KH == p.KW && (K == 2 || K == 3) && p.sh == 2 && p.sw == 2 && p.dh == 1 && p.dw == 1 &&
          p.pt == (K == 3) && p.pl == (K == 3) && p.W % 4 == 0 && p.H % 2 == 0 && p.OH == p.H / 2 && p.OW == p.W / 2))
        return false;
    if ((uintptr_t)X->data % (4 * sizeof(S)) || (uintptr_t)Y->data % (2 * sizeof(S))) return false;
    const size_t planes = (size_t)X->shape[0] * X->shape[1];
    const uint32_t quads = (uint32_t)(p.W / 4);
    int strip = 4;                                                    // output rows per thread (all of a strip's input rows are loaded up front)
    while (strip > 1 && planes * quads * (size_t)((p.OH + strip - 1) / strip) < (size_t)st->sm_count * 4096) strip /= 2;
    const uint32_t strips = (uint32_t)((p.OH + strip - 1) / strip);
    const size_t total = planes * quads * strips;
    if (total >= 0x7FFFFFFFull) return false;
    FastDiv by_quads, by_strips;
    by_quads.set(quads);
    by_strips.set(strips);
    const uint32_t grid = (uint32_t)((total + 255) / 256);
    const S* x = (const S*)X->data;
    S* y = (S*)Y->data;
#define TOPS_STRIPS(KK, SS) max_pool_stride2_strips<DT, KK, SS><<<grid, 256, 0, s>>>(x, y, p.H, p.W, p.OH, p.OW, quads, strips, by_quads, by_strips, (uint32_t)total)
    if (K == 2) { if (strip == 8) TOPS_STRIPS(2, 8); else if (strip == 4) TOPS_STRIPS(2, 4); else if (strip == 2) TOPS_STRIPS(2, 2); else TOPS_STRIPS(2, 1); }
    else        { if (strip == 8) TOPS_STRIPS(3, 8); else if (strip == 4) TOPS_STRIPS(3, 4); else if (strip == 2) TOPS_STRIPS(3, 2); else TOPS_STRIPS(3, 1); }
#undef TOPS_STRIPS
    return true;
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
