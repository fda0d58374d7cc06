// Conv2d over NCHW (tensor_ops.c:1036-1114).
//
// Entry point plus the exact path: one thread per output element reducing ic -> kh -> kw in
// double, bias added after the reduction -- the reference's own order, hence bit-identical for
// every dtype combination, group count, stride and dilation.  The implicit-GEMM tensor-core path
// (conv_tc.cu) takes the group == 1 float16 / bfloat16 / fp8 cases it supports.
#include "common.cuh"
#include "conv_common.cuh"

namespace tops {

template <bool EXACT_PRODUCTS>
__global__ void __launch_bounds__(256) conv_exact_kernel(const void* __restrict__ X, const void* __restrict__ Wt,
                                                          const void* __restrict__ Bias, void* __restrict__ Y,
                                                          int dx, int dw, int db, int dy, ConvGeom c, size_t total) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int ow = (int)(i % (size_t)c.OW);
        size_t t = i / (size_t)c.OW;
        const int oh = (int)(t % (size_t)c.OH); t /= (size_t)c.OH;
        const int m = (int)(t % (size_t)c.M);
        const size_t n = t / (size_t)c.M;
        const int cg = c.C / c.G, mg = c.M / c.G;
        const int c0 = (m / mg) * cg;
        const int h0 = oh * c.sh - c.pt, w0 = ow * c.sw - c.pl;
        double acc = 0.0;
        for (int ic = 0; ic < cg; ic++) {
            const size_t x_plane = ((n * c.C) + (size_t)(c0 + ic)) * c.H * c.W;
            const size_t w_base = ((size_t)m * cg + ic) * c.KH * c.KW;
            for (int kh = 0; kh < c.KH; kh++) {
                const int ih = h0 + kh * c.dh;
                for (int kw = 0; kw < c.KW; kw++) {
                    const int iw = w0 + kw * c.dw;
                    // padding taps contribute x = 0: adding 0 * w leaves the sum unchanged,
                    // except that it turns an Inf/NaN weight into NaN exactly as the reference does
                    double xv = 0.0;
                    if (ih >= 0 && ih < c.H && iw >= 0 && iw < c.W) xv = load_f64_rt(X, dx, x_plane + (size_t)ih * c.W + iw);
                    const double wv = load_f64_rt(Wt, dw, w_base + (size_t)kh * c.KW + kw);
                    if (EXACT_PRODUCTS) acc = fma(xv, wv, acc);
                    else acc = __dadd_rn(acc, __dmul_rn(xv, wv));
                }
            }
        }
        const double bias = Bias ? load_f64_rt(Bias, db, (size_t)m) : 0.0;
        store_f64_rt(Y, dy, i, __dadd_rn(acc, bias));
    }
}

bool conv_exact(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    const int grid = grid_for(Y->size, 256, st->sm_count, 8);
    const void* bias = (B && B->data) ? B->data : nullptr;
    const int db = bias ? (int)B->dtype : DTYPE_FLOAT32;
    const bool exact = dtype_exact_in_f32((int)X->dtype) && dtype_exact_in_f32((int)W->dtype);
    if (exact) conv_exact_kernel<true><<<grid, 256, 0, current_stream()>>>(X->data, W->data, bias, Y->data, (int)X->dtype,
                                                                          (int)W->dtype, db, (int)Y->dtype, c, Y->size);
    else conv_exact_kernel<false><<<grid, 256, 0, current_stream()>>>(X->data, W->data, bias, Y->data, (int)X->dtype,
                                                                     (int)W->dtype, db, (int)Y->dtype, c, Y->size);
    return TOPS_CHECK_LAUNCH("conv2d_forward");
}

bool conv_geometry(const char* name, const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvParams* params, ConvGeom* out) {
    if (!X || !W || !Y || !params || !X->data || !W->data || !Y->data || X->ndim != 4 || W->ndim != 4 || Y->ndim != 4 ||
        !params->pads || !params->strides || !params->dilations) {
        set_error(TOPS_ERR_INVALID, "%s: null argument or tensors that are not 4-D", name);
        zero_fill(Y);
        return false;
    }
    ConvGeom c;
    c.N = X->shape[0]; c.C = X->shape[1]; c.H = X->shape[2]; c.W = X->shape[3];
    c.M = W->shape[0]; c.KH = W->shape[2]; c.KW = W->shape[3];
    c.OH = Y->shape[2]; c.OW = Y->shape[3];
    c.pt = params->pads[0]; c.pl = params->pads[1];
    c.sh = params->strides[0]; c.sw = params->strides[1];
    c.dh = params->dilations[0]; c.dw = params->dilations[1];
    c.G = params->group;
    if (c.G < 1 || c.C % c.G || c.M % c.G || W->shape[1] != c.C / c.G || Y->shape[0] != c.N || Y->shape[1] != c.M ||
        c.sh < 1 || c.sw < 1 || (B && B->data && B->size < (size_t)c.M)) {
        set_error(TOPS_ERR_INVALID, "%s: inconsistent shapes or attributes", name);
        zero_fill(Y);
        return false;
    }
    *out = c;
    return true;
}

}  // namespace tops

using namespace tops;

TOPS_API void conv2d_forward(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, ConvParams* params) {
    ConvGeom c;
    if (!conv_geometry("conv2d_forward", X, W, B, Y, params, &c)) return;
    if (Y->size == 0) return;
    if (!conv_tensor_core(X, W, B, Y, c)) conv_exact(X, W, B, Y, c);
    finish_op();
}
