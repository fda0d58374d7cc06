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
// No cluster, no multicast: every CTA loads its own operands.  All waits are bounded.
#include "gemm_common.cuh"
#include "umma.cuh"
#include "elementwise.cuh"

#include <atomic>
#include <mutex>

namespace tops {

void count_tensor_core_launch();

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

// ---- kernel --------------------------------------------------------------------------------------------------------
constexpr int kBM = 128, kBN = 256, kRowBytes = 128, kStages = 4;
constexpr int kTileABytes = kBM * kRowBytes;       // 16 KB
constexpr int kTileBBytes = kBN * kRowBytes;       // 32 KB
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kTcThreads = 192;
constexpr int kStageRowWords = 36;                 // 32 words of payload + 4 of padding: conflict-free 16-byte accesses
constexpr size_t kTcSmemBytes = (size_t)kStages * kStageBytes + 1024 /*alignment slack*/ + 128 /*barriers*/ + 4 * kBN * 4 /*bias*/ +
                                4 * 32 * kStageRowWords * 4 /*output staging*/;

struct TcParams {
    int M, N;
    int k_blocks;          // K blocks of 128 bytes
    int k_step;            // elements per K block
    int tiles_m, tiles_n;
    void* Y;
    int dy;
    float alpha, beta;
    BiasView bias;
    int* status;           // device-visible word, set non-zero when a wait gave up
    int vec_store;         // Y base and row pitch are 16-byte aligned
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    // groups of 16 row blocks sweep all column blocks: concurrently running CTAs share A and B tiles in L2
    constexpr int kGroup = 16;
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int rows = min(kGroup, tiles_m - g * kGroup);
    tm = g * kGroup + r % rows;
    tn = r / rows;
}

template <bool FP8>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p,
               const uint32_t idesc) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + (size_t)kStages * kStageBytes);
    uint64_t* full = bars;                    // [kStages]  TMA -> MMA
    uint64_t* empty = bars + kStages;         // [kStages]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * kStages;  // [2]        MMA -> epilogue
    uint64_t* acc_empty = acc_full + 2;       // [2]        epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* bias_stage = (float*)(bars + 16);           // 4 warps x kBN floats
    uint32_t* out_stage = (uint32_t*)(bias_stage + 4 * kBN);   // 4 warps x 32 rows x kStageRowWords

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int total_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; s++) { umma::mbar_init(&full[s], 1); umma::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 2; b++) { umma::mbar_init(&acc_full[b], 1); umma::mbar_init(&acc_empty[b], 4); }
        *abort_flag = 0;
        umma::mbar_fence_init();
        umma::tma_prefetch_desc(&map_a);
        umma::tma_prefetch_desc(&map_b);
    }
    if (warp == 1) umma::tmem_alloc(tmem_slot, 512);
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!umma::mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
                    uint8_t* a_tile = tiles + (size_t)s * kStageBytes;
                    umma::mbar_expect_tx(&full[s], kStageBytes);
                    umma::tma_load_2d(a_tile, &map_a, &full[s], kb * p.k_step, tm * kBM);
                    umma::tma_load_2d(a_tile + kTileABytes, &map_b, &full[s], kb * p.k_step, tn * kBN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, local = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, local++) {
                const uint32_t buf = local & 1u, use = (local >> 1) & 1u;
                if (!umma::mbar_wait(&acc_empty[buf], use ^ 1u, abort_flag)) break;
                umma::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kBN;
                bool ok = true;
                for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                    const uint32_t s = it % kStages, ph = (it / kStages) & 1u;
                    if (!umma::mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                    umma::fence_after_sync();
                    const uint8_t* a_tile = tiles + (size_t)s * kStageBytes;
                    const uint64_t da = umma::smem_desc_k_major_sw128(a_tile);
                    const uint64_t db = umma::smem_desc_k_major_sw128(a_tile + kTileABytes);
                    #pragma unroll
                    for (int k = 0; k < kRowBytes / 32; k++)      // 32 bytes of K per instruction
                        umma::mma_ss<FP8>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, (kb | k) != 0);
                    umma::mma_commit(&empty[s]);                    // the stage is free once these MMAs retire
                }
                if (!ok) break;
                umma::mma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;                               // TMEM lanes this warp may read
        uint32_t local = 0;
        float* my_bias = bias_stage + quarter * kBN;                 // this warp's private copy: no cross-warp sync
        uint32_t* my_stage = out_stage + quarter * 32 * kStageRowWords;
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, local++) {
            const uint32_t buf = local & 1u, use = (local >> 1) & 1u;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            const int m = tm * kBM + quarter * 32 + lane;
            // beta * C for this tile, fetched while the tensor core is still working on it
            float row_bias = 0.0f;
            if (p.bias.mode == kBiasPerColumn) {
                __syncwarp();
                #pragma unroll
                for (int j = 0; j < kBN / 32; j++) {
                    const int n = tn * kBN + j * 32 + lane;
                    my_bias[j * 32 + lane] = n < p.N ? __fmul_rn(p.beta, (float)load_f64_rt(p.bias.ptr, p.bias.dtype, (size_t)n)) : 0.0f;
                }
                __syncwarp();
            } else if (p.bias.mode == kBiasScalar) {
                row_bias = __fmul_rn(p.beta, (float)load_f64_rt(p.bias.ptr, p.bias.dtype, 0));
            } else if (p.bias.mode == kBiasPerRow && m < p.M) {
                row_bias = __fmul_rn(p.beta, (float)load_f64_rt(p.bias.ptr, p.bias.dtype, (size_t)m));
            }
            if (!umma::mbar_wait(&acc_full[buf], use, abort_flag)) break;
            umma::fence_after_sync();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * kBN;
            #pragma unroll 1
            for (int c = 0; c < kBN / 32; c++) {
                uint32_t r[32];
                umma::tmem_load_32x32(t_row + (uint32_t)(c * 32), r);
                umma::tmem_load_wait();
                const int n0 = tn * kBN + c * 32;
                if (n0 < p.N) {                                    // warp-uniform
                    float v[32];
                    #pragma unroll
                    for (int j = 0; j < 32; j++) v[j] = __fadd_rn(__fmul_rn(p.alpha, __uint_as_float(r[j])), row_bias);
                    if (p.bias.mode == kBiasPerColumn) {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            const float4 b4 = *(const float4*)(my_bias + c * 32 + j);
                            v[j] = __fadd_rn(v[j], b4.x); v[j + 1] = __fadd_rn(v[j + 1], b4.y);
                            v[j + 2] = __fadd_rn(v[j + 2], b4.z); v[j + 3] = __fadd_rn(v[j + 3], b4.w);
                        }
                    } else if (p.bias.mode == kBiasMatrix && m < p.M) {
                        float cv[32];
                        if (p.bias.dtype == DTYPE_FLOAT32) {            // independent loads, issued back to back
                            #pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const long long ci = (n0 + j < p.N) ? bias_index(p.bias, m, n0 + j) : -1;
                                cv[j] = ci >= 0 ? __ldg((const float*)p.bias.ptr + ci) : 0.0f;
                            }
                        } else {
                            #pragma unroll
                            for (int j = 0; j < 32; j++) {
                                const long long ci = (n0 + j < p.N) ? bias_index(p.bias, m, n0 + j) : -1;
                                cv[j] = ci >= 0 ? (float)load_f64_rt(p.bias.ptr, p.bias.dtype, (size_t)ci) : 0.0f;
                            }
                        }
                        #pragma unroll
                        for (int j = 0; j < 32; j++) v[j] = __fmaf_rn(p.beta, cv[j], v[j]);
                    }
                    // Stage this warp's 32 x 32 chunk (already in output format) in shared memory,
                    // then write it out with every store instruction covering whole 128-byte lines.
                    uint32_t* my_rows = my_stage + lane * kStageRowWords;
                    if (p.dy == DTYPE_FLOAT32) {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *(uint4*)(my_rows + j) = make_uint4(__float_as_uint(v[j]), __float_as_uint(v[j + 1]),
                                                                 __float_as_uint(v[j + 2]), __float_as_uint(v[j + 3]));
                    } else if (p.dy == DTYPE_BFLOAT16) {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *(uint4*)(my_rows + (j >> 1)) = make_uint4(encode_bf16x2(v[j], v[j + 1]), encode_bf16x2(v[j + 2], v[j + 3]),
                                                                        encode_bf16x2(v[j + 4], v[j + 5]), encode_bf16x2(v[j + 6], v[j + 7]));
                    } else {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *(uint4*)(my_rows + (j >> 1)) = make_uint4(encode_f16x2(v[j], v[j + 1]), encode_f16x2(v[j + 2], v[j + 3]),
                                                                        encode_f16x2(v[j + 4], v[j + 5]), encode_f16x2(v[j + 6], v[j + 7]));
                    }
                    __syncwarp();
                    const int esize = p.dy == DTYPE_FLOAT32 ? 4 : 2;
                    const int lanes_per_row = esize * 2;                 // 16-byte pieces per 32-element row
                    const int rows_per_pass = 32 / lanes_per_row;
                    const int piece = lane % lanes_per_row;              // which 16 bytes of the row
                    const int elems_per_piece = 16 / esize;
                    const int n = n0 + piece * elems_per_piece;
                    #pragma unroll 1
                    for (int r0 = 0; r0 < 32; r0 += rows_per_pass) {
                        const int row = r0 + lane / lanes_per_row;
                        const int mr = tm * kBM + quarter * 32 + row;
                        if (mr >= p.M || n >= p.N) continue;
                        const uint4 val = *(const uint4*)(my_stage + row * kStageRowWords + piece * 4);
                        char* dst = (char*)p.Y + ((size_t)mr * p.N + n) * esize;
                        if (p.vec_store && n + elems_per_piece <= p.N) {
                            __stcs((uint4*)dst, val);
                        } else {
                            const uint32_t w[4] = {val.x, val.y, val.z, val.w};
                            for (int e = 0; e < elems_per_piece && n + e < p.N; e++) {
                                if (esize == 4) ((uint32_t*)dst)[e] = w[e];
                                else ((uint16_t*)dst)[e] = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
                            }
                        }
                    }
                    __syncwarp();
                }
            }
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) umma::mbar_arrive(&acc_empty[buf]);
        }
    }

    umma::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
    if (warp == 1) {
        umma::fence_after_sync();
        umma::tmem_dealloc(tmem_base, 512);
    }
}

// ---- host --------------------------------------------------------------------------------------------------------
static bool is_fp8(int dt) { return dt == DTYPE_FLOAT8_E4M3 || dt == DTYPE_FLOAT8_E5M2; }

bool gemm_tensor_core(const Tensor* A, const Tensor* B, Tensor* Y, const GemmShape& g, const BiasView& bias,
                      float alpha, float beta) {
    const int da = (int)A->dtype, db = (int)B->dtype, dy = (int)Y->dtype;
    const bool fp8 = is_fp8(da) && is_fp8(db);
    const bool half16 = (da == db) && (da == DTYPE_FLOAT16 || da == DTYPE_BFLOAT16);
    if (!fp8 && !half16) return false;
    if (dy != DTYPE_FLOAT32 && dy != DTYPE_BFLOAT16 && dy != DTYPE_FLOAT16) return false;
    if (g.transA != 0 || g.transB != 1) return false;                 // both operands K-major
    const int eb = fp8 ? 1 : 2;
    if (((size_t)g.K * eb) % 16 != 0 || ((uintptr_t)A->data & 15) || ((uintptr_t)B->data & 15)) return false;
    if (g.M < 1 || g.N < 1 || g.K < 1) return false;
    if (getenv("TOPS_DISABLE_TC")) return false;

    DeviceState* st = acquire_device();
    if (!st) return true;                                             // error already recorded

    const int k_step = kRowBytes / eb;
    CUtensorMap map_a, map_b;
    const uint64_t dims_a[2] = {(uint64_t)g.K, (uint64_t)g.M}, dims_b[2] = {(uint64_t)g.K, (uint64_t)g.N};
    const uint64_t strides_a[1] = {(uint64_t)g.lda * eb}, strides_b[1] = {(uint64_t)g.ldb * eb};
    const uint32_t box_a[2] = {(uint32_t)k_step, (uint32_t)kBM}, box_b[2] = {(uint32_t)k_step, (uint32_t)kBN};
    const bool f16 = da == DTYPE_FLOAT16;
    if (!make_tensor_map(&map_a, A->data, eb, fp8, f16, 2, dims_a, strides_a, box_a, nullptr) ||
        !make_tensor_map(&map_b, B->data, eb, fp8, f16, 2, dims_b, strides_b, box_b, nullptr))
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

    const uint32_t fa = fp8 ? (da == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (da == DTYPE_BFLOAT16 ? 1u : 0u);
    const uint32_t fb = fp8 ? (db == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (db == DTYPE_BFLOAT16 ? 1u : 0u);
    const uint32_t idesc = umma::instr_desc(fa, fb, kBM, kBN);
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < st->sm_count ? tiles : st->sm_count;
    cudaStream_t s = current_stream();
    if (fp8) {
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(gemm_tc_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes); attr = true; }
        gemm_tc_kernel<true><<<grid, kTcThreads, kTcSmemBytes, s>>>(map_a, map_b, p, idesc);
    } else {
        static bool attr = false;
        if (!attr) { cudaFuncSetAttribute(gemm_tc_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kTcSmemBytes); attr = true; }
        gemm_tc_kernel<false><<<grid, kTcThreads, kTcSmemBytes, s>>>(map_a, map_b, p, idesc);
    }
    TOPS_CHECK_LAUNCH("gemm_forward (tensor cores)");
    count_tensor_core_launch();
    return true;
}

static std::atomic<long long> g_tc_launches{0};
void count_tensor_core_launch() { g_tc_launches.fetch_add(1); }

}  // namespace tops

TOPS_API long long tops_tensor_core_launches(void) { return tops::g_tc_launches.load(); }
