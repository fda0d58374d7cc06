// Types shared by the Gemm / Conv entry points and their tensor-core kernels.
#pragma once

#include "common.cuh"

namespace tops {

struct GemmShape {
    int M, N, K;
    int lda, ldb;          // row lengths of A and B as stored
    int transA, transB;
};

// How C is broadcast over Y (tensor_ops.c:1194-1222).
enum BiasMode { kBiasNone = 0, kBiasScalar = 1, kBiasPerColumn = 2, kBiasPerRow = 3, kBiasMatrix = 4, kBiasZero = 5 };

struct BiasView {
    const void* ptr;
    int dtype;
    int mode;
    int rows, cols;        // last two dims of C for kBiasMatrix
};

// Element index of C for output (m, n); -1 when the reference would add zero.
__host__ __device__ inline long long bias_index(const BiasView& b, int m, int n) {
    switch (b.mode) {
        case kBiasScalar:    return 0;
        case kBiasPerColumn: return n;
        case kBiasPerRow:    return m;
        case kBiasMatrix: {
            const int r = b.rows == 1 ? 0 : m, c = b.cols == 1 ? 0 : n;
            return (r < b.rows && c < b.cols) ? (long long)r * b.cols + c : -1;
        }
        default:             return -1;
    }
}

// Scales of a fused DequantizeLinear -> Gemm / Conv -> QuantizeLinear sequence, all float32 in device
// memory so that nothing is read back to the host: the operand scales multiply the accumulator, the
// result scale divides it before rounding to an integer value and encoding (the reference's
// QuantizeLinear: rint(y / s), then the store of the output type).
struct EpilogueScales {
    const float* a_scale = nullptr;    // one value
    const float* b_scale = nullptr;    // one value, or one per output column
    int b_per_column = 0;
    const float* y_scale = nullptr;    // one value; only with 8-bit output types
};

// Convolution mode can hand its result to the NEXT quantised convolution directly: the value is
// quantised with that convolution's input scale and zero point (the arithmetic of
// quantize_linear_forward) and stored as a bfloat16 integer level in the channels-last, zero-padded
// (stride 2: space-to-depth) layout that convolution's tensor-core pass reads -- no float32 tensor in
// between.  `z` is cleared by the caller where the layout has padding cells.
struct LevelsOut {
    uint16_t* z = nullptr;             // [images][Hz][Wz][Cz]
    const float* scale = nullptr;      // one value
    const void* zero = nullptr;        // one int8 / uint8 value, or null for 0
    int zero_signed = 1;
    int S = 1, pt = 0, pl = 0, Hz = 0, Wz = 0, Cz = 0, C = 0;
};

BiasView make_bias_view(const Tensor* C, int M, int N);

// Element distances between consecutive problems of a batched launch (0: the operand is shared).
struct BatchStrides { size_t a = 0, b = 0, y = 0; };

// Exact double-accumulating path (any dtypes); `batches` equally spaced problems of one shape.
bool gemm_exact(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                float alpha, float beta, int batches = 1, BatchStrides batch = BatchStrides());

// Tensor-core path.  Returns false when the case is outside what it covers (caller falls back
// to the exact kernel, which is still a GPU kernel of this library).
// With `fused` (operand / result scales of a DQ -> Gemm -> Q sequence) 8-bit output types are accepted too.
// `batches` > 1: that many dense problems of shape g stored back to back in A, B and Y (no bias, no fusion,
// 16-bit or 8-bit float operands), one launch.
bool gemm_tensor_core(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                      float alpha, float beta, const EpilogueScales* fused = nullptr, int batches = 1);

}  // namespace tops
