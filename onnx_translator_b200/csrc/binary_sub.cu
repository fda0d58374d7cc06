// Sub with broadcasting: one instantiation set of binary_impl.cuh (tensor_ops.c:864-997).
#include "binary_impl.cuh"

TOPS_API void sub_forward(const Tensor* A, const Tensor* B, Tensor* O) {
    tops::binary_forward<tops::kSub>("sub_forward", A, B, O);
}
