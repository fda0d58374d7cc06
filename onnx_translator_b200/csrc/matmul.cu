// MatMul (tensor_ops.c:1546-1606): Y[..., m, n] = sum over k of A[..., m, k] * B[..., k, n], the leading
// (batch) dimensions broadcast numpy-style, operands of lower rank aligned to the right.
//
// Every batch is one Gemm without bias (alpha 1 leaves the sum untouched), so the two Gemm paths are reused:
//   * the exact kernel (double accumulation in increasing k, bit-identical to the reference) takes all
//     batches of a launch on grid.z when they are equally spaced, a stride of 0 standing for a broadcast
//     operand;
//   * the tensor-core kernel wants both operands K-major, so B ([K, N] per batch) is transposed into
//     scratch first -- 2 * K * N elements of traffic against M * N * K multiply-adds -- and is used for the
//     same input types and sizes as in gemm_forward; equal batches of 16-bit / 8-bit operands are one launch
//     (the batch is the third coordinate of the tensor maps), other batch patterns one launch per batch.
// A batched A against a single B is one Gemm with batches * M rows.
#include "common.cuh"
#include "gemm_common.cuh"

namespace tops {

template <typename T>
__global__ void __launch_bounds__(256) transpose_kn_kernel(const T* __restrict__ src, T* __restrict__ dst, int K, int N, size_t src_batch) {
    __shared__ T tile[32][33];
    const T* s = src + (size_t)blockIdx.z * src_batch;
    T* d = dst + (size_t)blockIdx.z * (size_t)K * (size_t)N;
    const int n0 = blockIdx.x * 32, k0 = blockIdx.y * 32;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    #pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int k = k0 + r, n = n0 + tx;
        if (k < K && n < N) tile[r][tx] = s[(size_t)k * N + n];
    }
    __syncthreads();
    #pragma unroll
    for (int r = ty; r < 32; r += 8) {
        const int n = n0 + r, k = k0 + tx;
        if (k < K && n < N) d[(size_t)n * K + k] = tile[tx][r];
    }
}

static bool transpose_kn(const void* src, void* dst, int elem_bytes, int K, int N, int batches, size_t src_batch, cudaStream_t s) {
    for (int first = 0; first < batches; first += 65535) {
        const int nb = batches - first < 65535 ? batches - first : 65535;
        const dim3 grid((N + 31) / 32, (K + 31) / 32, nb);
        const char* sp = (const char*)src + (size_t)first * src_batch * elem_bytes;
        char* dp = (char*)dst + (size_t)first * (size_t)K * N * elem_bytes;
        if (elem_bytes == 1) transpose_kn_kernel<uint8_t><<<grid, 256, 0, s>>>((const uint8_t*)sp, (uint8_t*)dp, K, N, src_batch);
        else if (elem_bytes == 2) transpose_kn_kernel<uint16_t><<<grid, 256, 0, s>>>((const uint16_t*)sp, (uint16_t*)dp, K, N, src_batch);
        else transpose_kn_kernel<uint32_t><<<grid, 256, 0, s>>>((const uint32_t*)sp, (uint32_t*)dp, K, N, src_batch);
    }
    return TOPS_CHECK_LAUNCH("matmul_forward (transpose B)");
}

// Element offset of the matrix an operand contributes to output batch `coords` (rank y_ndim - 2).
static size_t batch_offset(const Tensor* t, const int* coords, int y_ndim) {
    const int lead = t->ndim - 2, shift = y_ndim - t->ndim;
    size_t index = 0;
    for (int d = 0; d < lead; d++) index = index * (size_t)t->shape[d] + (size_t)(t->shape[d] == 1 ? 0 : coords[d + shift]);
    return index * (size_t)t->shape[t->ndim - 2] * (size_t)t->shape[t->ndim - 1];
}

// 1: every batch dimension of the operand equals the output's; 0: the operand is one matrix; -1: mixed.
static int batch_pattern(const Tensor* t, const Tensor* y) {
    const int shift = y->ndim - t->ndim;
    bool all_one = true, all_same = true;
    for (int d = 0; d < y->ndim - 2; d++) {
        const int mine = d >= shift ? t->shape[d - shift] : 1;
        if (mine != 1) all_one = false;
        if (mine != y->shape[d]) all_same = false;
    }
    return all_one ? 0 : (all_same ? 1 : -1);
}

static Tensor view_of(const Tensor* t, size_t element_offset) {
    Tensor v = *t;
    v.data = (char*)t->data + element_offset * (size_t)dtype_bytes((int)t->dtype);
    return v;
}

}  // namespace tops

using namespace tops;

TOPS_API void matmul_forward(const Tensor* A, const Tensor* B, Tensor* Y) {
    const char* name = "matmul_forward";
    if (!A || !B || !Y || !A->data || !B->data || !Y->data || A->ndim < 2 || B->ndim < 2 || Y->ndim < 2 || Y->ndim > 16 ||
        A->ndim > Y->ndim || B->ndim > Y->ndim) {
        set_error(TOPS_ERR_INVALID, "%s: null tensor, rank below 2, or an operand of higher rank than the output", name);
        zero_fill(Y);
        return;
    }
    const int M = A->shape[A->ndim - 2], K = A->shape[A->ndim - 1], N = B->shape[B->ndim - 1];
    bool ok = B->shape[B->ndim - 2] == K && Y->shape[Y->ndim - 2] == M && Y->shape[Y->ndim - 1] == N;
    size_t batches = 1;
    for (int d = 0; ok && d < Y->ndim - 2; d++) {
        const int ea = d - (Y->ndim - A->ndim) >= 0 ? A->shape[d - (Y->ndim - A->ndim)] : 1;
        const int eb = d - (Y->ndim - B->ndim) >= 0 ? B->shape[d - (Y->ndim - B->ndim)] : 1;
        ok = (ea == 1 || ea == Y->shape[d]) && (eb == 1 || eb == Y->shape[d]);
        batches *= (size_t)Y->shape[d];
    }
    if (!ok || batches > 0x7FFFFFFFull) {
        set_error(TOPS_ERR_INVALID, "%s: inner dimensions differ or the batch dimensions do not broadcast to the output's", name);
        zero_fill(Y);
        return;
    }
    if (Y->size == 0) return;
    DeviceState* st = acquire_device();
    if (!st) return;
    cudaStream_t s = current_stream();

    const int da = (int)A->dtype, db = (int)B->dtype, dy = (int)Y->dtype;
    const size_t a_mat = (size_t)M * K, b_mat = (size_t)K * N, y_mat = (size_t)M * N;
    int pa = batch_pattern(A, Y), pb = batch_pattern(B, Y);
    if (batches == 1) pa = pb = 0;

    // a batched A against one B: a single problem with batches * M rows
    int rows = M;
    size_t problems = batches;
    if (pb == 0 && pa == 1 && batches * (size_t)M <= 0x7FFFFFFFull) { rows = (int)(batches * (size_t)M); problems = 1; pa = 0; }

    GemmShape g;
    g.M = rows; g.N = N; g.K = K; g.lda = K; g.ldb = N; g.transA = 0; g.transB = 0;
    BiasView none;
    none.ptr = nullptr; none.dtype = DTYPE_FLOAT32; none.mode = kBiasNone; none.rows = none.cols = 1;

    // ---- tensor cores for the input types gemm_forward uses them for ---------------------------------
    const bool fp8 = (da == DTYPE_FLOAT8_E4M3 || da == DTYPE_FLOAT8_E5M2) && (db == DTYPE_FLOAT8_E4M3 || db == DTYPE_FLOAT8_E5M2);
    const bool half16 = da == db && (da == DTYPE_FLOAT16 || da == DTYPE_BFLOAT16);
    const bool big_f32 = da == DTYPE_FLOAT32 && db == DTYPE_FLOAT32 && K % 8 == 0 && (double)rows * N * K >= 134217728.0;
    const int eb = dtype_bytes(db);
    const bool float_out = dy == DTYPE_FLOAT32 || dy == DTYPE_BFLOAT16 || dy == DTYPE_FLOAT16;
    bool done = false;
    if ((fp8 || half16 || big_f32) && float_out && K > 0 && ((size_t)K * eb) % 16 == 0 && !getenv("TOPS_DISABLE_TC")) {
        const size_t b_sets = pb == 0 ? 1 : batches;                 // distinct B matrices (mixed broadcasting: one per output batch)
        void* bt = nullptr;
        if (cudaMallocAsync(&bt, b_sets * b_mat * eb, s) == cudaSuccess) {
            bool good = true;
            if (pb >= 0) good = transpose_kn(B->data, bt, eb, K, N, (int)b_sets, pb == 0 ? 0 : b_mat, s);
            GemmShape gt = g;
            gt.ldb = K; gt.transB = 1;
            done = good;
            int coords[16];
            size_t first = 0;
            if (good && problems > 1 && pa == 1 && pb == 1) {        // equal batches: one launch walks them all
                Tensor btv = *B;
                btv.data = bt;
                if (gemm_tensor_core(A, &btv, Y, gt, none, 1.0f, 0.0f, nullptr, (int)problems)) first = problems;
            }
            for (size_t i = first; good && i < problems; i++) {
                size_t rest = i;
                for (int d = Y->ndim - 3; d >= 0; d--) { coords[d] = (int)(rest % (size_t)Y->shape[d]); rest /= (size_t)Y->shape[d]; }
                const size_t a_off = problems == 1 ? 0 : batch_offset(A, coords, Y->ndim);
                const size_t b_off = problems == 1 ? 0 : batch_offset(B, coords, Y->ndim);
                if (pb < 0 && !transpose_kn((const char*)B->data + b_off * eb, (char*)bt + i * b_mat * eb, eb, K, N, 1, 0, s)) { done = false; break; }
                Tensor av = view_of(A, a_off), yv = view_of(Y, i * y_mat), btv = *B;
                btv.data = (char*)bt + (pb == 0 ? 0 : i * b_mat * eb);
                if (!gemm_tensor_core(&av, &btv, &yv, gt, none, 1.0f, 0.0f)) {
                    Tensor bv = view_of(B, b_off);                   // a case the tensor-core path does not cover (alignment)
                    if (!gemm_exact(&av, &bv, &yv, g, none, 1.0f, 0.0f)) { done = true; break; }
                }
            }
            cudaFreeAsync(bt, s);
        } else {
            cudaGetLastError();
        }
    }

    // ---- exact path ------------------------------------------------------------------------------------------
    if (!done) {
        if (pa >= 0 && pb >= 0) {
            BatchStrides strides;
            strides.a = pa ? a_mat : 0; strides.b = pb ? b_mat : 0; strides.y = y_mat;
            gemm_exact(A, B, Y, g, none, 1.0f, 0.0f, (int)problems, strides);
        } else {
            int coords[16];
            for (size_t i = 0; i < batches; i++) {
                size_t rest = i;
                for (int d = Y->ndim - 3; d >= 0; d--) { coords[d] = (int)(rest % (size_t)Y->shape[d]); rest /= (size_t)Y->shape[d]; }
                Tensor av = view_of(A, batch_offset(A, coords, Y->ndim)), bv = view_of(B, batch_offset(B, coords, Y->ndim)), yv = view_of(Y, i * y_mat);
                if (!gemm_exact(&av, &bv, &yv, g, none, 1.0f, 0.0f)) break;
            }
        }
    }
    finish_op();
}
