// Max with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:1367-1383).
#include "binary_impl.cuh"

TOPS_API void max_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kMax>("max_forward", A, B, O);
}
