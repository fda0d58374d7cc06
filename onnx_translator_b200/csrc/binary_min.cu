// Min with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:1386-1403).
#include "binary_impl.cuh"

TOPS_API void min_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kMin>("min_forward", A, B, O);
}
