// Types shared by the Conv2d entry point and its kernels.
#pragma once

#include "common.cuh"
#include "gemm_common.cuh"

namespace tops {

struct ConvGeom {
    int N, C, H, W;        // input
    int M, KH, KW;         // filters: [M, C / G, KH, KW]
    int OH, OW;            // output spatial size (chosen by the caller)
    int pt, pl;            // top / left padding (bottom / right only shape the output)
    int sh, sw, dh, dw;    // strides, dilations
    int G;                 // groups
};

bool conv_exact(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c);

// Implicit-GEMM tensor-core path; false when the case is outside what it covers.
bool conv_tensor_core(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c);

// The same path in two steps: eligibility and scratch sizes (no CUDA call), then the launches
// given two scratch buffers of at least xp_bytes / wt_bytes (16-byte aligned device memory).
struct ConvTcPlan {
    bool ok, fp8;
    int es, Hp, Wp, taps;
    size_t rows, xp_bytes, wt_bytes;
};
// `w_scale` (float32, one value per output channel, device memory): W holds int8 codes of a
// DequantizeLinear with zero point 0; the codes are widened exactly to X's 16-bit type while they
// are reordered and the scales are applied to the accumulator.
ConvTcPlan conv_tc_plan(const Tensor* X, const Tensor* W, const Tensor* Y, const ConvGeom& c, bool int8_weights = false);
bool conv_tc_run(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c, const ConvTcPlan& plan,
                 void* xp, void* wt, int* status, const float* w_scale = nullptr);

// The tensor-core step on operands that are already laid out: `xp` = activations [images][Hp][Wp][C]
// channels-last with every padding cell present, `wt` = filters [KH*KW][M][C]; output (n, m, oh, ow)
// for oh < OH, ow < OW reads rows (oh + kh*dil_h, ow + kw*dil_w).  C * es must be a multiple of 16.
struct ShiftedGemm {
    const void* xp = nullptr; const void* wt = nullptr;
    int es = 2; bool fp8 = false;
    int a_row_stride_bytes = 0;               // 0: C * es.  Smaller than that: row q also covers the cells after it (merged taps)
    unsigned a_format = 1, b_format = 1;      // tcgen05 operand formats (16-bit: 0 = float16, 1 = bfloat16; fp8: 0 = e4m3, 1 = e5m2)
    int images = 0, Hp = 0, Wp = 0, C = 0, M = 0, KH = 1, KW = 1, dil_h = 1, dil_w = 1, OH = 0, OW = 0;
    void* Y = nullptr; int dy = DTYPE_FLOAT32;
    const void* bias = nullptr; int bias_dtype = DTYPE_FLOAT32;
    int* status = nullptr;
    EpilogueScales fs;
    int relu = 0;
    const float* residual = nullptr;          // float32, shape of Y: added to the result before the optional Relu
    LevelsOut lv;                             // result as levels for the next quantised convolution (Y may then be null)
    int y_channels_last = 0;                  // Y is float32 [images][OH][OW][M] instead of NCHW
    int residual_channels_last = 0;           // the residual is [images][OH][OW][M]
};
bool shifted_gemm_launch(const ShiftedGemm& g);
// Whether the driver accepts the activation map of `g` (no launch): used to choose a layout before the filters are laid out.
bool shifted_gemm_map_ok(const ShiftedGemm& g);

// Fills a ConvGeom from the ABI arguments; false (with the error recorded) when they are inconsistent.
bool conv_geometry(const char* name, const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvParams* params, ConvGeom* c);

}  // namespace tops
