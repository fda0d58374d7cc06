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

}  // namespace tops
