// Fused forms of operator sequences that quantised graphs are made of.  Each entry point computes
// what the reference computes by calling its operators one after the other (nn/Operators.py:427-473
// for QuantizeLinear / DequantizeLinear, :475-548 for Conv, :613-669 for Gemm), without writing the
// dequantised operands or the unquantised result to memory:
//
//   tops_gemm_qdq_forward    DequantizeLinear(A), DequantizeLinear(B) -> Gemm -> [QuantizeLinear]
//   tops_conv2d_dqw_forward  DequantizeLinear(W, per output channel)  -> Conv
//
// The quantised codes go to the tensor cores as they are (fp8 codes as fp8 operands, int8 weight
// codes widened exactly to the activations' 16-bit type); the scales are applied to the fp32
// accumulator.  The difference to the unfused sequence is the accumulation order and the place of
// the scale multiplications, i.e. the same tolerance class as the tensor-core Gemm / Conv itself.
// Cases outside what the tensor-core kernels cover are refused (TOPS_ERR_UNSUPPORTED, output
// zero-filled): the caller then runs the unfused sequence, which covers everything.
#include "conv_common.cuh"
#include "gemm_common.cuh"

namespace tops {

static bool f32_device_values(const Tensor* t, size_t count) {
    return t && t->data && t->dtype == DTYPE_FLOAT32 && t->size == count;
}

}  // namespace tops

using namespace tops;

TOPS_API int tops_gemm_qdq_forward(const Tensor* A, const Tensor* a_scale, const Tensor* B, const Tensor* b_scale,
                                   const Tensor* C, const Tensor* y_scale, Tensor* Y,
                                   float alpha, float beta, int transA, int transB) {
    const char* name = "tops_gemm_qdq_forward";
    if (!A || !B || !Y || !A->data || !B->data || !Y->data || A->ndim != 2 || B->ndim != 2) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor or operands that are not 2-D", name);
        zero_fill(Y);
        return tops_last_error();
    }
    GemmShape g;
    g.transA = transA ? 1 : 0; g.transB = transB ? 1 : 0;
    g.M = transA ? A->shape[1] : A->shape[0];
    g.K = transA ? A->shape[0] : A->shape[1];
    g.N = transB ? B->shape[0] : B->shape[1];
    g.lda = A->shape[1]; g.ldb = B->shape[1];
    const int kb = transB ? B->shape[1] : B->shape[0];
    if (kb != g.K || Y->size != (size_t)g.M * (size_t)g.N) {
        set_error(TOPS_ERR_INVALID, "%s: inner dimensions differ or Y is not M x N", name);
        zero_fill(Y);
        return tops_last_error();
    }
    const bool fp8_in = (A->dtype == DTYPE_FLOAT8_E4M3 || A->dtype == DTYPE_FLOAT8_E5M2) &&
                        (B->dtype == DTYPE_FLOAT8_E4M3 || B->dtype == DTYPE_FLOAT8_E5M2);
    const bool eight_bit_out = Y->dtype == DTYPE_FLOAT8_E4M3 || Y->dtype == DTYPE_FLOAT8_E5M2 || Y->dtype == DTYPE_INT8 || Y->dtype == DTYPE_UINT8;
    if (!fp8_in || !f32_device_values(a_scale, 1) || !f32_device_values(b_scale, 1) ||
        (y_scale && (!f32_device_values(y_scale, 1) || !eight_bit_out)) || (!y_scale && eight_bit_out)) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: wants fp8 operands, one float32 scale each, and a float32 result scale exactly when Y is an 8-bit type", name);
        zero_fill(Y);
        return tops_last_error();
    }
    if (Y->size == 0) return TOPS_OK;
    EpilogueScales fs;
    fs.a_scale = (const float*)a_scale->data;
    fs.b_scale = (const float*)b_scale->data;
    fs.y_scale = y_scale ? (const float*)y_scale->data : nullptr;
    const BiasView bias = make_bias_view(C, g.M, g.N);
    if (!gemm_tensor_core(A, B, Y, g, bias, alpha, beta, &fs)) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: needs transA = 0, transB = 1, K a multiple of 16 and 16-byte aligned operands", name);
        zero_fill(Y);
        return tops_last_error();
    }
    finish_op();
    return TOPS_OK;
}

TOPS_API int tops_conv2d_dqw_forward(const Tensor* X, const Tensor* Wq, const Tensor* w_scale, const Tensor* B, Tensor* Y,
                                     ConvParams* params) {
    const char* name = "tops_conv2d_dqw_forward";
    ConvGeom c;
    if (!conv_geometry(name, X, Wq, B, Y, params, &c)) return tops_last_error();
    if (Wq->dtype != DTYPE_INT8 || !f32_device_values(w_scale, (size_t)c.M)) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: wants int8 filter codes and one float32 scale per output channel", name);
        zero_fill(Y);
        return tops_last_error();
    }
    if (Y->size == 0) return TOPS_OK;
    const ConvTcPlan plan = conv_tc_plan(X, Wq, Y, c, true);
    if (!plan.ok) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: covers group 1, stride 1, float16 / bfloat16 activations with C a multiple of 8, "
                                        "float32 / bfloat16 / float16 output", name);
        zero_fill(Y);
        return tops_last_error();
    }
    if (!acquire_device()) return tops_last_error();
    cudaStream_t s = current_stream();
    void *xp = nullptr, *wt = nullptr;
    if (cudaMallocAsync(&xp, plan.xp_bytes, s) != cudaSuccess) { cudaGetLastError(); set_error(TOPS_ERR_OOM, "%s: scratch", name); return tops_last_error(); }
    if (cudaMallocAsync(&wt, plan.wt_bytes, s) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeAsync(xp, s);
        set_error(TOPS_ERR_OOM, "%s: scratch", name);
        return tops_last_error();
    }
    const bool ok = conv_tc_run(X, Wq, B, Y, c, plan, xp, wt, device_status_word(), (const float*)w_scale->data);
    cudaFreeAsync(xp, s);
    cudaFreeAsync(wt, s);
    if (!ok) return tops_last_error();
    finish_op();
    return TOPS_OK;
}
