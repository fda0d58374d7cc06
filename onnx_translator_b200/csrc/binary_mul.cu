// Mul with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:864-997).
#include "binary_impl.cuh"

TOPS_API void mul_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kMul>("mul_forward", A, B, O);
}
