// Tensor-core Gemm for sm_100a: Y = alpha * A * B^T + beta * C with A [M,K] and B [N,K] both
// K-major (transA = 0, transB = 1), inputs fp16 / bf16 / fp8 (e4m3, e5m2), fp32 accumulation in
// tensor memory, output fp32 / bf16 / fp16.
//
// One persistent CTA per SM, 192 threads in three roles:
//   warp 0    TMA producer: 128-byte-swizzled tiles of A (128 x 128 B) and B (256 x 128 B) into a
//             4-stage shared-memory ring, one mbarrier per stage (expect_tx / complete_tx).
//   warp 1    MMA issuer: one lane issues tcgen05.mma (M 128, N 256, 32 bytes of K each) into one
//             of two 256-column accumulators in tensor memory; tcgen05.commit frees the stage and,
//             after the last K block, publishes the accumulator.
//   warps 2-5 epilogue: tcgen05.ld the accumulator (each warp its own 32-lane quarter), apply
//             alpha / beta * C, convert and store; then hand the accumulator back.  Because there
//             are two accumulators, the epilogue of tile i overlaps the main loop of tile i + 1.
// No cluster: every CTA loads its own operands.  All waits are bounded.
#include "tc_kernel.cuh"

#include <atomic>
#include <mutex>

namespace tops {


// ---- host: tensor maps -----------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

bool make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, bool is_fp8, bool is_fp16, int rank,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     const uint32_t* elem_strides) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t gdim[5], gstride[5];
    cuuint32_t bdim[5], estride[5];
    for (int i = 0; i < rank; i++) { gdim[i] = dims[i]; bdim[i] = box[i]; estride[i] = elem_strides ? elem_strides[i] : 1; }
    for (int i = 0; i + 1 < rank; i++) gstride[i] = strides_bytes[i];
    const CUtensorMapDataType dt = is_fp8 ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : (is_fp16 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16);
    (void)elem_bytes;
    const CUresult r = fn(out, dt, (cuuint32_t)rank, const_cast<void*>(base), gdim, gstride, bdim, estride,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

bool make_row_box_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    const uint32_t row_bytes = box_cols * (uint32_t)elem_bytes;
    if ((row_bytes != 32 && row_bytes != 64) || (elem_bytes != 2 && elem_bytes != 4)) return false;
    const cuuint64_t gdim[2] = {cols, rows}, gstride[1] = {cols * (uint64_t)elem_bytes};
    const cuuint32_t bdim[2] = {box_cols, box_rows}, estride[2] = {1, 1};
    const CUresult r = fn(out, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT16, 2, const_cast<void*>(base),
                          gdim, gstride, bdim, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          row_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// ---- host --------------------------------------------------------------------------------------------------------
static bool is_fp8(int dt) { return dt == DTYPE_FLOAT8_E4M3 || dt == DTYPE_FLOAT8_E5M2; }


// ---- float32 operands on the bfloat16 tensor cores -----------------------------------------------------------
// A float32 value is the exact sum of three bfloat16 values (8 + 8 + 8 significand bits):
// a = a1 + a2 + a3 with a1 = bf16(a), a2 = bf16(a - a1), a3 = bf16(a - a1 - a2).  The product a*b is
// then sum_ij a_i b_j; the three smallest of the nine terms (a2 b3, a3 b2, a3 b3) are below 2^-23 |a b|
// and are dropped, the other six are accumulated in float32 by one run of the tensor-core kernel whose
// K loop walks the plane pairs (smallest products first).  Error against the double-accumulating
// reference: about 3e-7 * sum_k |a_k b_k|, inside the 1e-6 gate used for every tensor-core result.
// Inf / NaN operands give NaN (Inf - Inf appears in the split).
__global__ void __launch_bounds__(256) split_f32_to_bf16x3(const float* __restrict__ src, uint16_t* __restrict__ planes,
                                                            size_t n, size_t plane_stride) {
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        const float4 v = *reinterpret_cast<const float4*>(src + i);          // n is a multiple of 8, src 16-byte aligned
        const float a[4] = {v.x, v.y, v.z, v.w};
        uint16_t p1[4], p2[4], p3[4];
        #pragma unroll
        for (int j = 0; j < 4; j++) {
            p1[j] = encode_bf16(a[j]);
            const float r1 = __fsub_rn(a[j], decode_bf16(p1[j]));
            p2[j] = encode_bf16(r1);
            const float r2 = __fsub_rn(r1, decode_bf16(p2[j]));
            p3[j] = encode_bf16(r2);
        }
        *reinterpret_cast<uint2*>(planes + i) = make_uint2(p1[0] | ((uint32_t)p1[1] << 16), p1[2] | ((uint32_t)p1[3] << 16));
        *reinterpret_cast<uint2*>(planes + plane_stride + i) = make_uint2(p2[0] | ((uint32_t)p2[1] << 16), p2[2] | ((uint32_t)p2[3] << 16));
        *reinterpret_cast<uint2*>(planes + 2 * plane_stride + i) = make_uint2(p3[0] | ((uint32_t)p3[1] << 16), p3[2] | ((uint32_t)p3[3] << 16));
    }
}

static bool gemm_split_f32(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                           float alpha, float beta) {
    DeviceState* st = acquire_device();
    if (!st) return true;
    cudaStream_t s = current_stream();
    const size_t a_elems = (size_t)g.M * g.K, b_elems = (size_t)g.N * g.K;
    uint16_t *ap = nullptr, *bp = nullptr;
    if (cudaMallocAsync((void**)&ap, a_elems * 6, s) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaMallocAsync((void**)&bp, b_elems * 6, s) != cudaSuccess) { cudaGetLastError(); cudaFreeAsync(ap, s); return false; }
    split_f32_to_bf16x3<<<grid_for(a_elems / 4, 256, st->sm_count, 8), 256, 0, s>>>((const float*)A->data, ap, a_elems, a_elems);
    split_f32_to_bf16x3<<<grid_for(b_elems / 4, 256, st->sm_count, 8), 256, 0, s>>>((const float*)B->data, bp, b_elems, b_elems);
    bool ok = TOPS_CHECK_LAUNCH("gemm_forward (float32 split)");

    const int k_step = kRowBytes / 2;
    CUtensorMap map_a, map_b;
    const uint64_t dims_a[3] = {(uint64_t)g.K, (uint64_t)g.M, 3}, dims_b[3] = {(uint64_t)g.K, (uint64_t)g.N, 3};
    const uint64_t strides_a[2] = {(uint64_t)g.K * 2, a_elems * 2}, strides_b[2] = {(uint64_t)g.K * 2, b_elems * 2};
    const uint32_t box_a[3] = {(uint32_t)k_step, (uint32_t)kBM, 1}, box_b[3] = {(uint32_t)k_step, (uint32_t)kBN, 1};
    ok = ok && make_tensor_map(&map_a, ap, 2, false, false, 3, dims_a, strides_a, box_a, nullptr) &&
         make_tensor_map(&map_b, bp, 2, false, false, 3, dims_b, strides_b, box_b, nullptr);
    if (ok) {
        TcParams p;
        p.M = g.M; p.N = g.N;
        p.cv.c_blocks = (g.K + k_step - 1) / k_step;
        p.k_blocks = 6 * p.cv.c_blocks;
        p.k_step = k_step;
        p.tiles_m = (g.M + kBM - 1) / kBM;
        p.tiles_n = (g.N + kBN - 1) / kBN;
        p.Y = Y->data; p.dy = (int)Y->dtype;
        p.alpha = alpha; p.beta = beta;
        p.bias = bias;
        p.status = device_status_word();
        p.vec_store = (((uintptr_t)Y->data & 15) == 0) && (((size_t)g.N * dtype_bytes((int)Y->dtype)) % 16 == 0);
        const uint32_t idesc = umma::instr_desc(1u, 1u, kBM, kBN);
        const int tiles = p.tiles_m * p.tiles_n;
        const int grid = tiles < st->sm_count ? tiles : st->sm_count;
        ok = ensure_dynamic_smem((const void*)tc_kernel<false, kModeSplit>, tc_smem_bytes(kModeSplit));
        if (ok) tc_kernel<false, kModeSplit><<<grid, tc_threads(kModeSplit), tc_smem_bytes(kModeSplit), s>>>(map_a, map_b, p, idesc, EpilogueMaps{});
        ok = ok && TOPS_CHECK_LAUNCH("gemm_forward (tensor cores, float32 split)");
        if (ok) count_tensor_core_launch();
    }
    cudaFreeAsync(ap, s);
    cudaFreeAsync(bp, s);
    return ok;
}

bool gemm_tensor_core(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                      float alpha, float beta, const EpilogueScales* fused, int batches) {
    const int da = (int)A->dtype, db = (int)B->dtype, dy = (int)Y->dtype;
    const bool fp8 = is_fp8(da) && is_fp8(db);
    const bool half16 = (da == db) && (da == DTYPE_FLOAT16 || da == DTYPE_BFLOAT16);
    // large float32 problems: three-way bfloat16 split (small ones keep the exact, bit-identical kernel)
    if (batches > 1 && (fused || bias.mode != kBiasNone || (da == DTYPE_FLOAT32 && db == DTYPE_FLOAT32))) return false;
    if (!fused && da == DTYPE_FLOAT32 && db == DTYPE_FLOAT32 && (dy == DTYPE_FLOAT32 || dy == DTYPE_BFLOAT16 || dy == DTYPE_FLOAT16) &&
        g.transA == 0 && g.transB == 1 && g.K % 8 == 0 && g.lda == g.K && g.ldb == g.K && !getenv("TOPS_DISABLE_TC") &&
        (((uintptr_t)A->data | (uintptr_t)B->data) & 15) == 0 && (double)g.M * g.N * g.K >= 134217728.0)
        return gemm_split_f32(A, B, Y, g, bias, alpha, beta);
    if (!fp8 && !half16) return false;
    const bool eight_bit_out = fused && (dy == DTYPE_FLOAT8_E4M3 || dy == DTYPE_FLOAT8_E5M2 || dy == DTYPE_INT8 || dy == DTYPE_UINT8);
    if (dy != DTYPE_FLOAT32 && dy != DTYPE_BFLOAT16 && dy != DTYPE_FLOAT16 && !eight_bit_out) return false;
    if (g.transA != 0 || g.transB != 1) return false;                 // both operands K-major
    const int eb = fp8 ? 1 : 2;
    if (((size_t)g.K * eb) % 16 != 0 || ((uintptr_t)A->data & 15) || ((uintptr_t)B->data & 15)) return false;
    if (g.M < 1 || g.N < 1 || g.K < 1) return false;
    if (getenv("TOPS_DISABLE_TC")) return false;

    DeviceState* st = acquire_device();
    if (!st) return true;                                             // error already recorded

    const int k_step = kRowBytes / eb;
    CUtensorMap map_a, map_b;
    // batches > 1: dense problems back to back, the batch index is the third map coordinate
    const uint64_t dims_a[3] = {(uint64_t)g.K, (uint64_t)g.M, (uint64_t)batches}, dims_b[3] = {(uint64_t)g.K, (uint64_t)g.N, (uint64_t)batches};
    const uint64_t strides_a[2] = {(uint64_t)g.lda * eb, (uint64_t)g.lda * eb * g.M}, strides_b[2] = {(uint64_t)g.ldb * eb, (uint64_t)g.ldb * eb * g.N};
    const uint32_t box_a[3] = {(uint32_t)k_step, (uint32_t)kBM, 1u}, box_b[3] = {(uint32_t)k_step, (uint32_t)kBN, 1u};
    const bool f16 = da == DTYPE_FLOAT16;
    const int rank = batches > 1 ? 3 : 2;
    if ((long long)((g.M + kBM - 1) / kBM) * ((g.N + kBN - 1) / kBN) * batches > 0x7FFFFFFFll) return false;
    if (!make_tensor_map(&map_a, A->data, eb, fp8, f16, rank, dims_a, strides_a, box_a, nullptr) ||
        !make_tensor_map(&map_b, B->data, eb, fp8, f16, rank, dims_b, strides_b, box_b, nullptr))
        return false;                                                 // let the exact kernel take it

    TcParams p;
    p.M = g.M; p.N = g.N;
    p.k_blocks = (g.K + k_step - 1) / k_step;
    p.k_step = k_step;
    p.tiles_m = (g.M + kBM - 1) / kBM;
    p.tiles_n = (g.N + kBN - 1) / kBN;
    p.Y = Y->data; p.dy = dy;
    p.alpha = alpha; p.beta = beta;
    p.bias = bias;
    p.status = device_status_word();
    p.vec_store = (((uintptr_t)Y->data & 15) == 0) && (((size_t)g.N * dtype_bytes(dy)) % 16 == 0);
    p.batches = batches;
    if (fused) p.fs = *fused;

    const uint32_t fa = fp8 ? (da == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (da == DTYPE_BFLOAT16 ? 1u : 0u);
    const uint32_t fb = fp8 ? (db == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (db == DTYPE_BFLOAT16 ? 1u : 0u);
    const uint32_t idesc = umma::instr_desc(fa, fb, kBM, kBN);
    const int tiles = p.tiles_m * p.tiles_n * batches;
    const int grid = tiles < st->sm_count ? tiles : st->sm_count;
    cudaStream_t s = current_stream();
    // few K blocks per tile: the epilogue is what the launch waits for, so it gets eight warps instead of four
    const bool short_k = p.k_blocks <= 8 && !getenv("TOPS_NO_SHORT_K_GEMM");
#define TOPS_GEMM_LAUNCH(F8, E)                                                                                                   \
    do {                                                                                                                          \
        static_assert(tc_smem_bytes(kModeGemm, E) <= 227 * 1024, "the variant's shared memory exceeds what a CTA can have");      \
        if (!ensure_dynamic_smem((const void*)tc_kernel<F8, kModeGemm, E>, tc_smem_bytes(kModeGemm, E))) return true;  /* error recorded */ \
        tc_kernel<F8, kModeGemm, E><<<grid, tc_threads(kModeGemm, E), tc_smem_bytes(kModeGemm, E), s>>>(map_a, map_b, p, idesc, EpilogueMaps{}); \
    } while (0)
    if (fp8 && short_k) TOPS_GEMM_LAUNCH(true, kEpiShortK);
    else if (fp8)       TOPS_GEMM_LAUNCH(true, kEpiPlain);
    else if (short_k)   TOPS_GEMM_LAUNCH(false, kEpiShortK);
    else                TOPS_GEMM_LAUNCH(false, kEpiPlain);
#undef TOPS_GEMM_LAUNCH
    TOPS_CHECK_LAUNCH("gemm_forward (tensor cores)");
    count_tensor_core_launch();
    return true;
}

static std::atomic<long long> g_tc_launches{0};
void count_tensor_core_launch() { g_tc_launches.fetch_add(1); }

}  // namespace tops

TOPS_API long long tops_tensor_core_launches(void) { return tops::g_tc_launches.load(); }
