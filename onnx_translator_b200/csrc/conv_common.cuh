// Types shared by the Conv2d entry point and its kernels.
#pragma once

#include "common.cuh"

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

// Fills a ConvGeom from the ABI arguments; false (with the error recorded) when they are inconsistent.
bool conv_geometry(const char* name, const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvParams* params, ConvGeom* c);

}  // namespace tops
