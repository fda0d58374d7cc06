// Pow with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:1355-1364).
#include "binary_impl.cuh"

TOPS_API void pow_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kPow>("pow_forward", A, B, O);
}
