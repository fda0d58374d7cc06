// Add with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:864-997).
#include "binary_impl.cuh"

TOPS_API void add_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kAdd>("add_forward", A, B, O);
}
