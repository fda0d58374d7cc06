// Gemm: Y = alpha * op(A) * op(B) + beta * C (tensor_ops.c:1167-1228).
//
// This file holds the entry point, the bias-broadcast rules and the exact path: a shared-memory
// tiled kernel that accumulates in double in increasing-k order, i.e. the reference's own
// summation order, for every dtype combination.  Its results are bit-identical to the reference.
// Tensor-core paths (gemm_tc.cu) take over for the 16-bit and 8-bit float inputs they support.
#include "common.cuh"
#include "gemm_common.cuh"

namespace tops {

constexpr int kTile = 64;      // output tile edge
constexpr int kTileK = 16;
constexpr int kPerThread = 4;  // 16 x 16 threads, 4 x 4 outputs each

template <bool EXACT_PRODUCTS>
__global__ void __launch_bounds__(256) gemm_exact_kernel(const void* __restrict__ A, const void* __restrict__ B,
                                                          void* __restrict__ Y, int da, int db, int dy,
                                                          GemmShape g, BiasView bias, double alpha, double beta, BatchStrides batch) {
    // blockIdx.z walks equally spaced problems (MatMul batches); a stride of 0 re-reads a broadcast operand
    const size_t a_base = (size_t)blockIdx.z * batch.a, b_base = (size_t)blockIdx.z * batch.b, y_base = (size_t)blockIdx.z * batch.y;
    __shared__ double sa[kTileK][kTile + 1];
    __shared__ double sb[kTileK][kTile + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    double acc[kPerThread][kPerThread] = {};

    for (int k0 = 0; k0 < g.K; k0 += kTileK) {
        // stage a kTileK x kTile slab of op(A) and op(B), zero beyond the edges
        for (int e = threadIdx.x; e < kTileK * kTile; e += 256) {
            int kk, mm;
            if (g.transA) { mm = e % kTile; kk = e / kTile; } else { kk = e % kTileK; mm = e / kTileK; }
            const int m = m0 + mm, k = k0 + kk;
            double v = 0.0;
            if (m < g.M && k < g.K) v = load_f64_rt(A, da, a_base + (g.transA ? (size_t)k * g.lda + m : (size_t)m * g.lda + k));
            sa[kk][mm] = v;
        }
        for (int e = threadIdx.x; e < kTileK * kTile; e += 256) {
            int kk, nn;
            if (g.transB) { kk = e % kTileK; nn = e / kTileK; } else { nn = e % kTile; kk = e / kTile; }
            const int n = n0 + nn, k = k0 + kk;
            double v = 0.0;
            if (n < g.N && k < g.K) v = load_f64_rt(B, db, b_base + (g.transB ? (size_t)n * g.ldb + k : (size_t)k * g.ldb + n));
            sb[kk][nn] = v;
        }
        __syncthreads();
        #pragma unroll
        for (int kk = 0; kk < kTileK; kk++) {
            double av[kPerThread], bv[kPerThread];
            #pragma unroll
            for (int i = 0; i < kPerThread; i++) { av[i] = sa[kk][ty * kPerThread + i]; bv[i] = sb[kk][tx * kPerThread + i]; }
            #pragma unroll
            for (int i = 0; i < kPerThread; i++)
                #pragma unroll
                for (int j = 0; j < kPerThread; j++) {
                    // products of float32-exact inputs are exact in double, so the fused form
                    // rounds exactly like "multiply, then add"; otherwise keep two roundings
                    if (EXACT_PRODUCTS) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
                    else acc[i][j] = __dadd_rn(acc[i][j], __dmul_rn(av[i], bv[j]));
                }
        }
        __syncthreads();
    }
    #pragma unroll
    for (int i = 0; i < kPerThread; i++)
        #pragma unroll
        for (int j = 0; j < kPerThread; j++) {
            const int m = m0 + ty * kPerThread + i, n = n0 + tx * kPerThread + j;
            if (m >= g.M || n >= g.N) continue;
            double r = __dmul_rn(alpha, acc[i][j]);
            if (bias.mode != kBiasNone) {
                const long long ci = bias_index(bias, m, n);
                const double cv = ci >= 0 ? load_f64_rt(bias.ptr, bias.dtype, (size_t)ci) : 0.0;
                r = __dadd_rn(r, __dmul_rn(beta, cv));
            }
            store_f64_rt(Y, dy, y_base + (size_t)m * g.N + n, r);
        }
}

// Few outputs, long reductions (a classifier layer on one image: 1 x 4096 times 4096 x 10): the 64 x 64 tiling
// above would run one CTA that stops at two barriers every 16 steps of k.  Here a CTA owns 4 x 16 outputs; 192 of
// its threads copy the next 128-deep slab of both operands into shared memory while the other 64 walk the current
// slab, one output each, in increasing k -- the reference's summation order, so the result stays bit-identical.
constexpr int kSkM = 4, kSkN = 16, kSkK = 128;

// F32_IN: both operands are float32 -- the copy threads then issue all of their loads before they use any (with the
// run-time dtype switch every load waited for the one before it, and a slab took several memory latencies to arrive:
// the K = 4096 classifier of the small CNN went from about 90 to 60 us; what is left is the chain of 4096 dependent
// double-precision additions the reference's summation order imposes -- copying further ahead changed nothing).
template <bool EXACT_PRODUCTS, bool F32_IN>
__global__ void __launch_bounds__(256) gemm_skinny_kernel(const void* __restrict__ A, const void* __restrict__ B,
                                                           void* __restrict__ Y, int da, int db, int dy,
                                                           GemmShape g, BiasView bias, double alpha, double beta, BatchStrides batch) {
    const size_t a_base = (size_t)blockIdx.z * batch.a, b_base = (size_t)blockIdx.z * batch.b, y_base = (size_t)blockIdx.z * batch.y;
    __shared__ double sa[2][kSkM][kSkK];
    __shared__ double sb[2][kSkN][kSkK + 1];
    const int m0 = blockIdx.y * kSkM, n0 = blockIdx.x * kSkN;
    const bool computes = threadIdx.x < kSkM * kSkN;
    const int i = threadIdx.x / kSkN, j = threadIdx.x % kSkN;
    const int chunks = (g.K + kSkK - 1) / kSkK;
    auto fill = [&](int chunk, int buf, int first, int step) {
        const int k0 = chunk * kSkK;
        if constexpr (F32_IN) {
            constexpr int kTotal = (kSkM + kSkN) * kSkK, kMost = (kTotal + 191) / 192;      // elements per copy thread at most
            float v[kMost];
            #pragma unroll
            for (int t = 0; t < kMost; t++) {
                const int e = first + t * step, row = e / kSkK, kk = e - row * kSkK, k = k0 + kk;
                v[t] = 0.0f;
                if (e < kTotal && k < g.K) {
                    if (row < kSkM) {
                        const int m = m0 + row;
                        if (m < g.M) v[t] = __ldg((const float*)A + a_base + (g.transA ? (size_t)k * g.lda + m : (size_t)m * g.lda + k));
                    } else {
                        const int n = n0 + row - kSkM;
                        if (n < g.N) v[t] = __ldg((const float*)B + b_base + (g.transB ? (size_t)n * g.ldb + k : (size_t)k * g.ldb + n));
                    }
                }
            }
            #pragma unroll
            for (int t = 0; t < kMost; t++) {
                const int e = first + t * step, row = e / kSkK, kk = e - row * kSkK;
                if (e >= kTotal) break;
                if (row < kSkM) sa[buf][row][kk] = (double)v[t];
                else sb[buf][row - kSkM][kk] = (double)v[t];
            }
            return;
        }
        for (int e = first; e < (kSkM + kSkN) * kSkK; e += step) {
            const int row = e / kSkK, kk = e - row * kSkK, k = k0 + kk;
            double v = 0.0;
            if (row < kSkM) {
                const int m = m0 + row;
                if (m < g.M && k < g.K) v = load_f64_rt(A, da, a_base + (g.transA ? (size_t)k * g.lda + m : (size_t)m * g.lda + k));
                sa[buf][row][kk] = v;
            } else {
                const int n = n0 + row - kSkM;
                if (n < g.N && k < g.K) v = load_f64_rt(B, db, b_base + (g.transB ? (size_t)n * g.ldb + k : (size_t)k * g.ldb + n));
                sb[buf][row - kSkM][kk] = v;
            }
        }
    };
    fill(0, 0, threadIdx.x, 256);
    __syncthreads();
    double acc = 0.0;
    for (int c = 0; c < chunks; c++) {
        if (computes) {
            const double* pa = sa[c & 1][i];
            const double* pb = sb[c & 1][j];
            #pragma unroll 8
            for (int kk = 0; kk < kSkK; kk++) {
                if (EXACT_PRODUCTS) acc = fma(pa[kk], pb[kk], acc);
                else acc = __dadd_rn(acc, __dmul_rn(pa[kk], pb[kk]));
            }
        } else if (c + 1 < chunks) {
            fill(c + 1, (c + 1) & 1, threadIdx.x - kSkM * kSkN, 256 - kSkM * kSkN);
        }
        __syncthreads();
    }
    const int m = m0 + i, n = n0 + j;
    if (!computes || m >= g.M || n >= g.N) return;
    double r = __dmul_rn(alpha, acc);
    if (bias.mode != kBiasNone) {
        const long long ci = bias_index(bias, m, n);
        const double cv = ci >= 0 ? load_f64_rt(bias.ptr, bias.dtype, (size_t)ci) : 0.0;
        r = __dadd_rn(r, __dmul_rn(beta, cv));
    }
    store_f64_rt(Y, dy, y_base + (size_t)m * g.N + n, r);
}

BiasView make_bias_view(const Tensor* C, int M, int N) {
    BiasView b;
    b.ptr = nullptr; b.dtype = DTYPE_FLOAT32; b.mode = kBiasNone; b.rows = 1; b.cols = 1;
    if (!C || !C->data) return b;
    b.ptr = C->data;
    b.dtype = (int)C->dtype;
    if (C->size == 1) { b.mode = kBiasScalar; return b; }
    if (C->ndim == 1) {
        if (C->shape[0] == N) b.mode = kBiasPerColumn;        // tested first: wins when M == N
        else if (C->shape[0] == M) b.mode = kBiasPerRow;
        else b.mode = kBiasZero;                               // the reference adds beta * 0
        return b;
    }
    b.mode = kBiasMatrix;
    b.rows = C->shape[C->ndim - 2];
    b.cols = C->shape[C->ndim - 1];
    // the shapes the Python layer produces for a 1-D C -- (1, N) and (M, 1) -- index exactly like
    // the per-column / per-row cases (only when C holds nothing beyond those two dimensions)
    if (C->size == (size_t)b.rows * (size_t)b.cols) {
        if (b.rows == 1 && b.cols == N) b.mode = kBiasPerColumn;
        else if (b.cols == 1 && b.rows == M) b.mode = kBiasPerRow;
    }
    return b;
}

bool gemm_exact(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                float alpha, float beta, int batches, BatchStrides batch) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    const bool exact = dtype_exact_in_f32((int)A->dtype) && dtype_exact_in_f32((int)B->dtype);
    const size_t ea = (size_t)dtype_bytes((int)A->dtype), eb = (size_t)dtype_bytes((int)B->dtype), ey = (size_t)dtype_bytes((int)Y->dtype);
    // too few 64 x 64 tiles to fill the GPU and a reduction long enough to matter: the 4 x 16 tiling
    const bool skinny = g.K >= 4 * kSkK && (size_t)((g.M + kTile - 1) / kTile) * ((g.N + kTile - 1) / kTile) * batches < (size_t)st->sm_count / 2;
    for (int first = 0; first < batches; first += 65535) {         // grid.z limit
        const int nb = batches - first < 65535 ? batches - first : 65535;
        dim3 grid((g.N + kTile - 1) / kTile, (g.M + kTile - 1) / kTile, nb);
        const void* a = (const char*)A->data + (size_t)first * batch.a * ea;
        const void* b = (const char*)B->data + (size_t)first * batch.b * eb;
        void* y = (char*)Y->data + (size_t)first * batch.y * ey;
        if (skinny) {
            const dim3 sgrid((g.N + kSkN - 1) / kSkN, (g.M + kSkM - 1) / kSkM, nb);
            const bool f32 = A->dtype == DTYPE_FLOAT32 && B->dtype == DTYPE_FLOAT32;
#define TOPS_SKINNY(EX, F) gemm_skinny_kernel<EX, F><<<sgrid, 256, 0, current_stream()>>>(a, b, y, (int)A->dtype, (int)B->dtype, (int)Y->dtype, g, bias, \
                                                                                       (double)alpha, (double)beta, batch)
            if (exact && f32) TOPS_SKINNY(true, true);
            else if (exact)   TOPS_SKINNY(true, false);
            else if (f32)     TOPS_SKINNY(false, true);
            else              TOPS_SKINNY(false, false);
#undef TOPS_SKINNY
            continue;
        }
        if (exact) gemm_exact_kernel<true><<<grid, 256, 0, current_stream()>>>(a, b, y, (int)A->dtype, (int)B->dtype, (int)Y->dtype, g, bias,
                                                                               (double)alpha, (double)beta, batch);
        else gemm_exact_kernel<false><<<grid, 256, 0, current_stream()>>>(a, b, y, (int)A->dtype, (int)B->dtype, (int)Y->dtype, g, bias,
                                                                          (double)alpha, (double)beta, batch);
    }
    return TOPS_CHECK_LAUNCH("gemm_forward");
}

}  // namespace tops

using namespace tops;

TOPS_API void gemm_forward(const Tensor* A, const Tensor* B, const Tensor* C, Tensor* Y,
                           float alpha, float beta, int transA, int transB) {
    if (!A || !B || !Y || !A->data || !B->data || !Y->data || A->ndim != 2 || B->ndim != 2) {
        set_error(TOPS_ERR_INVALID, "gemm_forward: null tensor or operands that are not 2-D");
        zero_fill(Y);
        return;
    }
    GemmShape g;
    g.transA = transA ? 1 : 0; g.transB = transB ? 1 : 0;
    g.M = transA ? A->shape[1] : A->shape[0];
    g.K = transA ? A->shape[0] : A->shape[1];
    g.N = transB ? B->shape[0] : B->shape[1];
    g.lda = A->shape[1]; g.ldb = B->shape[1];
    const int kb = transB ? B->shape[1] : B->shape[0];
    if (kb != g.K || Y->size != (size_t)g.M * (size_t)g.N) {
        set_error(TOPS_ERR_INVALID, "gemm_forward: inner dimensions differ or Y is not M x N");
        zero_fill(Y);
        return;
    }
    if (Y->size == 0) return;
    const BiasView bias = make_bias_view(C, g.M, g.N);
    if (!gemm_tensor_core(A, B, Y, g, bias, alpha, beta))       // false: not a case it covers
        gemm_exact(A, B, Y, g, bias, alpha, beta);
    finish_op();
}
