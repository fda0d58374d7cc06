// The persistent tcgen05 kernel shared by Gemm and Conv2d (see gemm_tc.cu for the role layout).
#pragma once

#include "gemm_common.cuh"
#include "umma.cuh"
#include "elementwise.cuh"
#include "qdq_math.cuh"

namespace tops {

// ---- kernel --------------------------------------------------------------------------------------------------------
constexpr int kBM = 128, kBN = 256, kRowBytes = 128, kStages = 4;
constexpr int kTileABytes = kBM * kRowBytes;       // 16 KB
constexpr int kTileBBytes = kBN * kRowBytes;       // 32 KB
constexpr int kStageBytes = kTileABytes + kTileBBytes;
constexpr int kStageRowWords = 36;                 // 32 words of payload + 4 of padding: conflict-free 16-byte accesses

// Per mode: the convolution's K loops are short and its epilogue is what bounds it, so it trades one pipeline
// stage for more epilogue warps -- more loads and stores in flight per SM.  A warp may only read the quarter of
// tensor memory given by its index modulo 4, so the warps that share a quarter take alternate column chunks.
constexpr int kModeGemm = 0, kModeConv = 1, kModeSplit = 2;
// The plain and the levels-only epilogue stage nothing but their per-channel constants and have room for four stages
// (a 3 x 3 convolution over 256 channels has 36 K blocks per tile, and the copy latency is what the multiplier waits
// for: the levels-only layers of a ResNet-50-shaped graph gained 6-14 % from the fourth stage); the residual variant
// was measured slower with four (76 -> 86 us for its one layer there) and the row-linear epilogue (EPI bit 2) stages
// its tiles in shared memory: three.
// The row-linear epilogue (EPI bit 2) with residual AND levels keeps two stages: its layers have short K loops and are
// bound by the epilogue, and the third stage's room holds staging and the per-channel constants instead.
// Gemm mode, EPI bit 3 (short reductions: a handful of K blocks per tile): the epilogue bounds such a launch -- four warps
// carry every output of a 128 x 256 tile through scale, convert and store -- so that variant runs eight epilogue warps
// (two per quarter of the tile's rows, alternate column chunks) and gives one pipeline stage for their staging.
__host__ __device__ constexpr int tc_stages(int mode, int epi = 0) {
    return mode != kModeConv ? ((epi & 8) ? 3 : kStages) : (epi & 5) == 0 ? kStages : (epi & 7) == 7 ? 2 : 3;
}
// Epilogue warps: 4 for the Gemm modes.  Convolution mode is bound by its epilogue (short K loops, strided NCHW
// stores, residual loads, quantisation to levels), so it handles 16 accumulator columns at a time -- half the
// registers per thread -- and runs 16 epilogue warps, or 12 where the residual is compiled in (its prefetch
// registers do not fit the 96-register budget of 18 warps without spilling; measured slower).
__host__ __device__ constexpr int tc_epilogue_warps(int mode, int epi = 0) { return mode != kModeConv ? ((epi & 8) ? 8 : 4) : ((epi & 4) ? 16 : (epi & 1) ? 12 : 16); }
// Row-linear epilogue (EPI bit 2): bytes of shared memory each epilogue warp stages its tiles in -- 32 rows x 64 bytes of
// float32 output, the same of residual input, 32 rows x 32 bytes of levels -- and where the warps' barriers live.
constexpr int kRowsOutBytes = 2048, kRowsResBytes = 2048, kRowsLevBytes = 1024, kRowsBarBytes = 1024;
__host__ __device__ constexpr int rows_warp_bytes(int epi) { return kRowsOutBytes + ((epi & 1) ? kRowsResBytes : 0) + ((epi & 2) ? kRowsLevBytes : 0); }
// ... and of the per-channel constants it keeps there for the whole launch: x_scale * w_scale[n] and beta * bias[n] of up
// to kRowsMaxChannels output channels, computed once per CTA instead of once per value.
constexpr int kRowsMaxChannels = 2048, kRowsColumnBytes = 2 * kRowsMaxChannels * 4;
__host__ __device__ constexpr int tc_chunk_columns(int mode) { return mode == kModeConv ? 16 : 32; }
__host__ __device__ constexpr int tc_threads(int mode, int epi = 0) { return 64 + 32 * tc_epilogue_warps(mode, epi); }
__host__ __device__ constexpr size_t tc_smem_bytes(int mode, int epi = 0) {
    if (mode == kModeConv && (epi & 4))
        return (size_t)tc_stages(mode, epi) * kStageBytes + 1024 /*alignment slack*/ + kRowsBarBytes + kRowsColumnBytes + (size_t)tc_epilogue_warps(mode, epi) * rows_warp_bytes(epi);
    return (size_t)tc_stages(mode, epi) * kStageBytes + 1024 /*alignment slack*/ + 384 /*barriers*/ +
           (size_t)tc_epilogue_warps(mode, epi) * kBN * 4 /*bias*/ + (size_t)tc_epilogue_warps(mode, epi) * kBN * 4 /*column scales*/ +
           (mode == kModeConv ? 0 : tc_epilogue_warps(mode, epi) * 32 * kStageRowWords * 4) /*output staging (row-major outputs only)*/;
}

// Convolution as shifted GEMMs over a zero-padded channels-last copy of the input: row q of the
// GEMM is the padded position (n, oh, ow) = (q / plane, (q % plane) / Wp, q % Wp); filter tap
// (kh, kw) reads rows q + kh * dil_h * Wp + kw * dil_w.  Rows with oh >= OH or ow >= OW are
// computed and dropped.
struct ConvView {
    int Wp, plane;         // padded width, padded plane size Hp * Wp
    int images, OH, OW, OC;
    int c_blocks;          // K blocks per filter tap
    int KW, dil_h, dil_w;
    FastDiv by_plane, by_Wp;   // row index -> (image, padded row, padded column) without integer divisions
};

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
    uint32_t stage_tx = kStageBytes;   // bytes the two copies of a pipeline stage deliver (less when the B box is narrower than kBN)
    int stages = 0;                    // pipeline stages in use (0: as many as the kernel variant reserves room for) ...
    uint32_t stage_bytes = kStageBytes;   // ... of this many bytes each: a narrower B box leaves room for more, smaller stages
    int kb_per_stage = 1;              // K blocks (of stage_tx bytes each, back to back) that share one stage and its pair of barriers
    int batches = 1;       // Gemm mode: independent problems of one shape; the tensor maps are then 3-D
                           // (K, rows, batch) and Y holds the results back to back
    ConvView cv;           // convolution mode only
    EpilogueScales fs;
    int relu = 0;          // clamp the result at zero before it is stored (v > 0 ? v : 0)
    const float* residual = nullptr;   // convolution mode: float32 tensor of the output's shape added before the clamp
    LevelsOut lv;                      // convolution mode: also / instead write the result as levels for the next convolution
    int acc_buffers = 2;               // accumulator buffers in tensor memory: 2 x 256 columns, 4 x 128 (N <= 128) or 8 x 64 (N <= 64)
    int epilogue_groups = 2;           // sixteen epilogue warps: how many tiles they finish at a time (1, 2 or 4 groups)
    int y_cl = 0;                      // convolution mode: Y (float32) is stored channels-last [N][OH][OW][OC] instead of NCHW
    int res_cl = 0;                    // convolution mode: the residual is stored channels-last
};

__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    // groups of 16 row blocks sweep all column blocks: concurrently running CTAs share A and B tiles in L2
    if (tiles_n == 1) { tm = tile; tn = 0; return; }              // one column block: no integer divisions
    constexpr int kGroup = 16;
    const int per_group = kGroup * tiles_n;
    const int g = tile / per_group, r = tile - g * per_group;
    const int rows = min(kGroup, tiles_m - g * kGroup);
    tm = g * kGroup + r % rows;
    tn = r / rows;
}

// MODE 0: Gemm.  MODE 1: Conv2d as shifted GEMMs (ConvView).  MODE 2: Gemm on float32 operands that
// were split into three bfloat16 planes each (see gemm_tc.cu); the K loop walks six plane pairs.

// EPI (convolution mode only) selects the epilogue extras that are compiled in, so that a kernel
// carries registers only for what it uses: bit 0 = residual operand, bit 1 = levels output.
// Bit 2 (convolutions whose GEMM row IS the output pixel: 1 x 1, no padding, and everything float32 channels-last):
// the epilogue moves its tiles with the copy engine -- residual in, float32 and levels out -- through per-warp
// staging in shared memory, so no thread issues a global load or store of its own.
// Requantisation to levels in the epilogues: q = v * (1 / s) with the CORRECTLY ROUNDED reciprocal is within 2^-23 |q| of
// v / s (two roundings of 2^-24 each), so rounding q decides rint(v / s) for every value further than that from a
// tie; the margin tested is twice the bound.  (The elementwise kernels use the approximate reciprocal and 2^-19.)
constexpr float kLevelsTieMargin = 2.3841858e-7f;      // 2^-22
__device__ __forceinline__ float levels_reciprocal(float s) {
    return fabsf(s) < 8.5e37f ? __frcp_rn(s) : __int_as_float(0x7FC00000);      // NaN: every value takes the exact division
}
constexpr int kEpiPlain = 0, kEpiResidual = 1, kEpiLevels = 2, kEpiRows = 4, kEpiShortK = 8;     // the last: Gemm mode only

// Tensor maps of the row-linear epilogue (unused by every other variant): [rows][OC] matrices in boxes of 32 rows x 16 columns.
struct EpilogueMaps { CUtensorMap y, res, lv; };

template <bool FP8, int MODE, int EPI = kEpiPlain>
__global__ void __launch_bounds__(tc_threads(MODE, EPI), 1)
tc_kernel(const __grid_constant__ CUtensorMap map_a, const __grid_constant__ CUtensorMap map_b, const TcParams p,
               const uint32_t idesc, const __grid_constant__ EpilogueMaps em) {
    // Launched with programmatic stream serialisation the CTAs are scheduled while the previous kernel of the stream drains
    // (one SM at a time, as its CTAs leave); nothing here touches memory before that kernel has completed.
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    constexpr int kSt = tc_stages(MODE, EPI), kEpi = tc_epilogue_warps(MODE, EPI);
    // Sixteen epilogue warps work as groups, one per accumulator buffer: consecutive tiles of the CTA are finished by
    // different groups, so the latency chain of one tile's epilogue (accumulator ready -> tensor memory load ->
    // arithmetic -> stores) overlaps the next tiles' instead of following it.  Two buffers of 256 columns and two
    // groups of eight warps normally; layers with at most 128 output channels get FOUR buffers of 128 columns and four
    // groups of four warps (one per quarter of the tile's rows): twice as many tiles in flight, and a warp meets each
    // tile's fixed work (row decode, barrier hand-offs) once per four column chunks instead of once per two.
    // More buffers than groups matter as much as the groups: a group that has finished a tile finds the next accumulator
    // already complete instead of waiting for the copy and multiply roles to refill the buffer it has just released.
    const int n_buf = kEpi >= 16 ? p.acc_buffers : 2;                    // 2, 4 or 8 buffers of 256, 128 or 64 columns
    const int epi_groups = kEpi >= 16 ? p.epilogue_groups : 1, epi_per_group = kEpi / epi_groups;
    const uint32_t acc_stride = 512u / (uint32_t)n_buf;
    // tile counter -> (buffer, phase, group) without a division
    const uint32_t buf_mask = (uint32_t)n_buf - 1u, buf_shift = n_buf == 8 ? 3u : n_buf == 4 ? 2u : 1u, group_mask = (uint32_t)epi_groups - 1u;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* tiles = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(tiles + (size_t)kSt * kStageBytes);
    // Stages: the variant reserves kSt * kStageBytes; a layer whose filter box is narrow cuts that room into more, smaller
    // stages (short K loops wait on the copy latency, and more stages in flight hide more of it).
    constexpr int kMaxStages = 8;
    const uint32_t n_st = p.stages > 0 ? (uint32_t)p.stages : (uint32_t)kSt;
    const uint32_t stage_bytes = p.stages > 0 ? p.stage_bytes : (uint32_t)kStageBytes;
    uint64_t* full = bars;                    // [kMaxStages]  TMA -> MMA
    uint64_t* empty = bars + kMaxStages;      // [kMaxStages]  MMA -> TMA
    uint64_t* acc_full = bars + 2 * kMaxStages;   // [8]    MMA -> epilogue
    uint64_t* acc_empty = acc_full + 8;       // [8]    epilogue -> MMA
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 8);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* bias_stage = (float*)(bars + 34);                   // kEpi warps x kBN floats
    float* scale_stage = bias_stage + kEpi * kBN;              // kEpi warps x kBN floats
    uint32_t* out_stage = (uint32_t*)(scale_stage + kEpi * kBN);   // 4 warps x 32 rows x kStageRowWords (not in convolution mode)
    constexpr bool kRows = MODE == kModeConv && (EPI & kEpiRows) != 0;
    // row-linear epilogue: [barrier block of 1 KB: pipeline barriers, then one residual barrier per epilogue warp][per-warp staging]
    uint64_t* res_bars = bars + 40;
    float* col_scale = (float*)((uint8_t*)bars + kRowsBarBytes);    // [kRowsMaxChannels], then the biases
    float* col_bias = col_scale + kRowsMaxChannels;
    uint8_t* rows_stage = (uint8_t*)bars + kRowsBarBytes + kRowsColumnBytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_per_batch = p.tiles_m * p.tiles_n;
    const int total_tiles = MODE == kModeGemm ? tiles_per_batch * p.batches : tiles_per_batch;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < n_st; s++) { umma::mbar_init(&full[s], 1); umma::mbar_init(&empty[s], 1); }
        for (int b = 0; b < 8; b++) { umma::mbar_init(&acc_full[b], 1); umma::mbar_init(&acc_empty[b], (uint32_t)epi_per_group); }
        if constexpr (kRows) for (int w = 0; w < kEpi; w++) umma::mbar_init(&res_bars[w], 1);
        *abort_flag = 0;
        umma::mbar_fence_init();
        umma::tma_prefetch_desc(&map_a);
        umma::tma_prefetch_desc(&map_b);
    }
    if (warp == 1) umma::tmem_alloc(tmem_slot, 512);
    if constexpr (kRows) {
        float alpha = p.alpha;
        if (p.fs.a_scale) alpha = __fmul_rn(alpha, __ldg(p.fs.a_scale));
        for (int n = threadIdx.x; n < p.N; n += blockDim.x) {
            col_scale[n] = p.fs.b_per_column ? __fmul_rn(alpha, __ldg(p.fs.b_scale + n)) : alpha;
            col_bias[n] = p.bias.mode == kBiasPerColumn ? __fmul_rn(p.beta, __ldg((const float*)p.bias.ptr + n)) : 0.0f;
        }
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            // One thread feeds the whole pipeline, so every instruction of this loop is on the critical path of a K
            // block: stage index, phase and filter tap are carried as counters -- an integer division by a run-time
            // value costs this thread more than the multiplies of a short K block take.
            uint32_t s = 0, ph = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x) {
                int tm, tn;
                const int bt = (MODE == kModeGemm && p.batches > 1) ? tile / tiles_per_batch : 0;
                tile_coords(tile - bt * tiles_per_batch, p.tiles_m, p.tiles_n, tm, tn);
                int cb = 0, tap = 0, kw = 0, shift = 0;             // channel block inside the tap / plane pair, tap, its column, its row shift
                // the two copies of K block kb, into the stage memory at a_tile, completing on bar
                auto copy_k_block = [&](int kb, uint8_t* a_tile, uint64_t* bar) {
                    if constexpr (MODE == kModeSplit) {
                        // smallest products first: (a3 b1) (a2 b2) (a1 b3) (a2 b1) (a1 b2) (a1 b1)
                        const int seg = tap;
                        const int plane_a = (0x001012 >> (4 * seg)) & 0xF, plane_b = (0x010210 >> (4 * seg)) & 0xF;
                        umma::tma_load_3d(a_tile, &map_a, bar, cb * p.k_step, tm * kBM, plane_a);
                        umma::tma_load_3d(a_tile + kTileABytes, &map_b, bar, cb * p.k_step, tn * kBN, plane_b);
                    } else if constexpr (MODE == kModeConv) {
                        umma::tma_load_2d(a_tile, &map_a, bar, cb * p.k_step, tm * kBM + shift);
                        umma::tma_load_3d(a_tile + kTileABytes, &map_b, bar, cb * p.k_step, tn * kBN, tap);
                    } else if (p.batches > 1) {
                        umma::tma_load_3d(a_tile, &map_a, bar, kb * p.k_step, tm * kBM, bt);
                        umma::tma_load_3d(a_tile + kTileABytes, &map_b, bar, kb * p.k_step, tn * kBN, bt);
                    } else {
                        umma::tma_load_2d(a_tile, &map_a, bar, kb * p.k_step, tm * kBM);
                        umma::tma_load_2d(a_tile + kTileABytes, &map_b, bar, kb * p.k_step, tn * kBN);
                    }
                    if constexpr (MODE != kModeGemm) {
                        if (++cb == p.cv.c_blocks) {                // next filter tap (next plane pair in split mode)
                            cb = 0; tap++;
                            if constexpr (MODE == kModeConv) {
                                shift += p.cv.dil_w;
                                if (++kw == p.cv.KW) { kw = 0; shift += p.cv.dil_h * p.cv.Wp - p.cv.KW * p.cv.dil_w; }
                            }
                        }
                    }
                };
                int kb = 0;
                if (MODE == kModeConv && p.kb_per_stage == 2) {
                    // narrow layers: two K blocks share a stage and its pair of barriers (one round trip for both)
                    for (; kb + 2 <= p.k_blocks; kb += 2) {
                        if (!umma::mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
                        uint8_t* a_tile = tiles + (size_t)s * stage_bytes;
                        umma::mbar_expect_tx(&full[s], 2u * p.stage_tx);
                        copy_k_block(kb, a_tile, &full[s]);
                        copy_k_block(kb + 1, a_tile + p.stage_tx, &full[s]);
                        if (++s == n_st) { s = 0; ph ^= 1u; }
                    }
                }
                for (; kb < p.k_blocks; kb++) {
                    if (!umma::mbar_wait(&empty[s], ph ^ 1u, abort_flag)) break;
                    uint8_t* a_tile = tiles + (size_t)s * stage_bytes;
                    umma::mbar_expect_tx(&full[s], p.stage_tx);
                    copy_k_block(kb, a_tile, &full[s]);
                    if (++s == n_st) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t s = 0, ph = 0, local = 0;
            for (int tile = blockIdx.x; tile < total_tiles && !*abort_flag; tile += gridDim.x, local++) {
                const uint32_t buf = local & buf_mask, use = (local >> buf_shift) & 1u;
                if (!umma::mbar_wait(&acc_empty[buf], use ^ 1u, abort_flag)) break;
                umma::fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * acc_stride;
                bool ok = true;
                auto multiply_k_block = [&](const uint8_t* a_tile, uint32_t accumulate) {
                    const uint64_t da = umma::smem_desc_k_major_sw128(a_tile);
                    const uint64_t db = umma::smem_desc_k_major_sw128(a_tile + kTileABytes);
                    #pragma unroll
                    for (int k = 0; k < kRowBytes / 32; k++)          // 32 bytes of K per instruction
                        umma::mma_ss<FP8>(d_tmem, da + (uint64_t)(k * 2), db + (uint64_t)(k * 2), idesc, accumulate | (uint32_t)k);
                };
                int kb = 0;
                if (MODE == kModeConv && p.kb_per_stage == 2) {
                    for (; kb + 2 <= p.k_blocks; kb += 2) {
                        if (!umma::mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                        umma::fence_after_sync();
                        const uint8_t* a_tile = tiles + (size_t)s * stage_bytes;
                        multiply_k_block(a_tile, (uint32_t)kb);
                        multiply_k_block(a_tile + p.stage_tx, 1u);
                        umma::mma_commit(&empty[s]);                // the stage is free once these MMAs retire
                        if (++s == n_st) { s = 0; ph ^= 1u; }
                    }
                }
                for (; ok && kb < p.k_blocks; kb++) {
                    if (!umma::mbar_wait(&full[s], ph, abort_flag)) { ok = false; break; }
                    umma::fence_after_sync();
                    multiply_k_block(tiles + (size_t)s * stage_bytes, (uint32_t)kb);
                    umma::mma_commit(&empty[s]);                    // the stage is free once these MMAs retire
                    if (++s == n_st) { s = 0; ph ^= 1u; }
                }
                if (!ok) break;
                umma::mma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;                               // TMEM lanes this warp may read
        const int epi = warp - 2;                                   // 0 .. kEpi-1
        const int group = epi / epi_per_group, eg = epi - group * epi_per_group;     // group: which accumulator buffer's tiles this warp finishes
        const int kChunkStep = epi_per_group / 4;                   // warps of a group that share a quarter alternate chunks
        constexpr int kW = tc_chunk_columns(MODE);                  // accumulator columns a warp handles at a time
        const int first_chunk = eg >> 2;
        uint32_t local = 0;
        if constexpr (kRows) {
            // ---- row-linear epilogue: every global access is a tile copy ------------------------------------------------
            constexpr bool with_res = (EPI & kEpiResidual) != 0, with_lv = (EPI & kEpiLevels) != 0;
            uint8_t* st_out = rows_stage + (size_t)epi * rows_warp_bytes(EPI);
            uint8_t* st_res = st_out + kRowsOutBytes;
            uint8_t* st_lv = st_res + (with_res ? kRowsResBytes : 0);
            uint64_t* res_bar = &res_bars[epi];
            uint32_t res_phase = 0;
            float lv_scale = 0.0f, lv_inv = 0.0f, lv_zero = 0.0f;
            if constexpr (with_lv) {
                lv_scale = __ldg(p.lv.scale);
                lv_inv = levels_reciprocal(lv_scale);
                if (p.lv.zero) lv_zero = p.lv.zero_signed ? (float)*(const int8_t*)p.lv.zero : (float)*(const uint8_t*)p.lv.zero;
            }
            const float lo = p.lv.zero_signed ? -128.0f : 0.0f, hi = p.lv.zero_signed ? 127.0f : 255.0f;
            const float lo_z = __fsub_rn(lo, lv_zero), hi_z = __fsub_rn(hi, lv_zero);
            // this lane's 16-byte chunks inside the staged boxes (row = lane)
            uint32_t off64[4], off32[2];
            #pragma unroll
            for (int j = 0; j < 4; j++) off64[j] = umma::swizzled_chunk<64>((uint32_t)lane, (uint32_t)j);
            #pragma unroll
            for (int j = 0; j < 2; j++) off32[j] = umma::swizzled_chunk<32>((uint32_t)lane, (uint32_t)j);
            bool alive = true;
            for (int tile = blockIdx.x; tile < total_tiles && alive; tile += gridDim.x, local++) {
                const uint32_t buf = local & buf_mask, use = (local >> buf_shift) & 1u;
                if ((int)(local & group_mask) != group) continue;
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const int row0 = tm * kBM + quarter * 32;             // first of this warp's 32 rows = output pixels
                if constexpr (with_res) {                              // the first chunk's residual travels while the tensor core works
                    if (lane == 0 && tn * kBN + first_chunk * kW < p.N) {
                        umma::mbar_expect_tx(res_bar, kRowsResBytes);
                        umma::tma_load_2d(st_res, &em.res, res_bar, tn * kBN + first_chunk * kW, row0);
                    }
                }
                if (!umma::mbar_wait(&acc_full[buf], use, abort_flag)) break;
                umma::fence_after_sync();
                const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * acc_stride;
                #pragma unroll 1
                for (int c = first_chunk; c < kBN / kW; c += kChunkStep) {
                    const int n0 = tn * kBN + c * kW;
                    if (n0 >= p.N) break;                              // p.N is a multiple of kW here
                    uint32_t r[kW];
                    umma::tmem_load_chunk<kW>(t_row + (uint32_t)(c * kW), r);
                    float v[kW];
                    umma::tmem_load_wait();
                    // per-channel constants from shared memory (every lane reads the same 16 bytes: a broadcast)
                    #pragma unroll
                    for (int j = 0; j < kW; j += 4) {
                        const float4 s4 = *(const float4*)(col_scale + n0 + j);
                        v[j] = __fmul_rn(s4.x, __uint_as_float(r[j]));         v[j + 1] = __fmul_rn(s4.y, __uint_as_float(r[j + 1]));
                        v[j + 2] = __fmul_rn(s4.z, __uint_as_float(r[j + 2])); v[j + 3] = __fmul_rn(s4.w, __uint_as_float(r[j + 3]));
                    }
                    if (p.bias.mode == kBiasPerColumn) {
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) {
                            const float4 b4 = *(const float4*)(col_bias + n0 + j);
                            v[j] = __fadd_rn(v[j], b4.x); v[j + 1] = __fadd_rn(v[j + 1], b4.y);
                            v[j + 2] = __fadd_rn(v[j + 2], b4.z); v[j + 3] = __fadd_rn(v[j + 3], b4.w);
                        }
                    }
                    if constexpr (with_res) {
                        if (!umma::mbar_wait(res_bar, res_phase, abort_flag)) { alive = false; break; }
                        res_phase ^= 1u;
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) {
                            const float4 r4 = *(const float4*)(st_res + off64[j >> 2]);
                            v[j] = __fadd_rn(v[j], r4.x); v[j + 1] = __fadd_rn(v[j + 1], r4.y);
                            v[j + 2] = __fadd_rn(v[j + 2], r4.z); v[j + 3] = __fadd_rn(v[j + 3], r4.w);
                        }
                        __syncwarp();                                  // every lane has read its row: the buffer may be refilled
                        const int c_next = c + kChunkStep;
                        if (lane == 0 && c_next < kBN / kW && tn * kBN + c_next * kW < p.N) {
                            umma::mbar_expect_tx(res_bar, kRowsResBytes);
                            umma::tma_load_2d(st_res, &em.res, res_bar, tn * kBN + c_next * kW, row0);
                        }
                    }
                    if (p.relu) {
                        #pragma unroll
                        for (int j = 0; j < kW; j++) v[j] = fmaxf(v[j], 0.0f);
                    }
                    uint32_t packed[kW / 2];
                    if constexpr (with_lv) {
                        #pragma unroll
                        for (int j0 = 0; j0 < kW; j0 += 8) {
                            float level[8];
                            bool decided = true;
                            #pragma unroll
                            for (int e = 0; e < 8; e++) {
                                const float q = __fmul_rn(v[j0 + e], lv_inv);
                                const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                                decided = decided & (fmaf(fabsf(q), kLevelsTieMargin, fabsf(__fsub_rn(q, rq))) < 0.5f);
                                level[e] = fminf(fmaxf(rq, lo_z), hi_z);
                            }
                            if (!decided) {                             // rare: redo only the values the fast rounding could not decide
                                #pragma unroll
                                for (int e = 0; e < 8; e++) {
                                    const float q = __fmul_rn(v[j0 + e], lv_inv);
                                    const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                                    if (!(fmaf(fabsf(q), kLevelsTieMargin, fabsf(__fsub_rn(q, rq))) < 0.5f))
                                        level[e] = quantize_level_exact(v[j0 + e], lv_scale, lv_zero, p.lv.zero_signed);
                                }
                            }
                            #pragma unroll
                            for (int e = 0; e < 8; e += 2)
                                packed[(j0 + e) >> 1] = __byte_perm(__float_as_uint(level[e]), __float_as_uint(level[e + 1]), 0x7632);
                        }
                    }
                    // the previous chunk's stores must have read the staging buffers before they are overwritten
                    if (lane == 0) umma::bulk_wait_read();
                    __syncwarp();
                    if (p.Y != nullptr) {
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) *(float4*)(st_out + off64[j >> 2]) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                    }
                    if constexpr (with_lv) {
                        #pragma unroll
                        for (int j = 0; j < kW / 8; j++)
                            *(uint4*)(st_lv + off32[j]) = make_uint4(packed[4 * j], packed[4 * j + 1], packed[4 * j + 2], packed[4 * j + 3]);
                    }
                    umma::fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        if (p.Y != nullptr) umma::tma_store_2d(&em.y, st_out, n0, row0);
                        if constexpr (with_lv) umma::tma_store_2d(&em.lv, st_lv, n0, row0);
                        umma::bulk_commit();
                    }
                }
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) umma::mbar_arrive(&acc_empty[buf]);
            }
            if (lane == 0) umma::bulk_wait_all();                   // the staging buffers outlive every store that reads them
        } else {
        float* my_bias = bias_stage + epi * kBN;                     // this warp's private copy: no cross-warp sync
        uint32_t* my_stage = out_stage + epi * 32 * kStageRowWords;       // one staging area per epilogue warp
        float* my_scale = scale_stage + epi * kBN;
        int staged_tn = -1;
        float alpha = p.alpha;
        if (p.fs.a_scale) alpha = __fmul_rn(alpha, __ldg(p.fs.a_scale));
        if (p.fs.b_scale && !p.fs.b_per_column) alpha = __fmul_rn(alpha, __ldg(p.fs.b_scale));
        const float y_scale = p.fs.y_scale ? __ldg(p.fs.y_scale) : 0.0f;
        const float y_inv = y_scale != 0.0f ? __frcp_rn(y_scale) : 0.0f;     // y / s as y * (1 / s): off by an ulp at most, like the accumulation itself
        // scale and zero point of the levels output: fetched once, not once per column chunk (each fetch is a
        // dependent global load in front of the chunk's arithmetic)
        float lv_scale = 0.0f, lv_inv = 0.0f, lv_zero = 0.0f;
        if constexpr (MODE == kModeConv && (EPI & kEpiLevels) != 0) {
            lv_scale = __ldg(p.lv.scale);
            lv_inv = levels_reciprocal(lv_scale);
            if (p.lv.zero) lv_zero = p.lv.zero_signed ? (float)*(const int8_t*)p.lv.zero : (float)*(const uint8_t*)p.lv.zero;
        }
        for (int tile = blockIdx.x; tile < total_tiles; tile += gridDim.x, local++) {
            const uint32_t buf = local & buf_mask, use = (local >> buf_shift) & 1u;
            if ((int)(local & group_mask) != group) continue;       // another group's tile
            int tm, tn;
            const int bt = (MODE == kModeGemm && p.batches > 1) ? tile / tiles_per_batch : 0;
            tile_coords(tile - bt * tiles_per_batch, p.tiles_m, p.tiles_n, tm, tn);
            const int m = tm * kBM + quarter * 32 + lane;
            // beta * C for this tile, fetched while the tensor core is still working on it
            float row_bias = 0.0f;
            const bool restage = tn != staged_tn;                 // per-column operands of a column block are staged once
            staged_tn = tn;
            if (p.bias.mode == kBiasPerColumn && restage) {
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
            if (p.fs.b_per_column && restage) {
                __syncwarp();
                #pragma unroll
                for (int j = 0; j < kBN / 32; j++) {
                    const int n = tn * kBN + j * 32 + lane;
                    my_scale[j * 32 + lane] = n < p.N ? __fmul_rn(alpha, __ldg(p.fs.b_scale + n)) : 0.0f;
                }
                __syncwarp();
            }
            // convolution mode: where this lane's row goes in the NCHW output, and the residual values
            // of the first column chunk, requested before the accumulator is even complete
            bool conv_row = false;
            size_t conv_base = 0, plane_out = 0, cl_base = 0;
            uint16_t* levels_row = nullptr;
            float res_next[kW];
            constexpr bool with_res = MODE == kModeConv && (EPI & kEpiResidual) != 0;
            if constexpr (MODE == kModeConv) {
                const int img = (int)p.cv.by_plane.div((uint32_t)m), rem = m - img * p.cv.plane;
                const int oh = (int)p.cv.by_Wp.div((uint32_t)rem), ow = rem - oh * p.cv.Wp;
                conv_row = img < p.cv.images && oh < p.cv.OH && ow < p.cv.OW;
                plane_out = (size_t)p.cv.OH * p.cv.OW;
                conv_base = ((size_t)img * p.cv.OC + (size_t)tn * kBN) * plane_out + (size_t)oh * p.cv.OW + ow;
                // the same element in a channels-last tensor: the row's channels are contiguous
                cl_base = (((size_t)img * p.cv.OH + oh) * p.cv.OW + ow) * (size_t)p.cv.OC + (size_t)tn * kBN;
                if constexpr ((EPI & kEpiLevels) != 0) {
                    // where this row's levels go: it is input pixel (oh, ow) of the next convolution -- worked out
                    // once per tile, not once per column chunk (two integer divisions per lane)
                    int A = oh + p.lv.pt, B = ow + p.lv.pl, slot = 0;
                    if (p.lv.S == 2) { slot = ((A & 1) * 2 + (B & 1)) * p.lv.C; A >>= 1; B >>= 1; }
                    levels_row = p.lv.z + (((size_t)img * p.lv.Hz + A) * p.lv.Wz + B) * p.lv.Cz + slot + tn * kBN;
                }
            }
            auto fetch_residual = [&](int chunk, float (&dst)[kW]) {
                if (p.res_cl) {                                    // kW consecutive floats of this row
                    const float* src = p.residual + cl_base + chunk * kW;
                    const int left = p.N - (tn * kBN + chunk * kW);
                    if (conv_row && left >= kW && (p.N & 3) == 0) {
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) {
                            const float4 v4 = __ldg((const float4*)(src + j));
                            dst[j] = v4.x; dst[j + 1] = v4.y; dst[j + 2] = v4.z; dst[j + 3] = v4.w;
                        }
                    } else {
                        #pragma unroll
                        for (int j = 0; j < kW; j++) dst[j] = (conv_row && j < left) ? __ldg(src + j) : 0.0f;
                    }
                    return;
                }
                const float* src = p.residual + conv_base + (size_t)(chunk * kW) * plane_out;
                #pragma unroll
                for (int j = 0; j < kW; j++)
                    dst[j] = (conv_row && tn * kBN + chunk * kW + j < p.N) ? __ldg(src + (size_t)j * plane_out) : 0.0f;
            };
            if constexpr (with_res) fetch_residual(first_chunk, res_next);
            if (!umma::mbar_wait(&acc_full[buf], use, abort_flag)) break;
            umma::fence_after_sync();
            const uint32_t t_row = tmem_base + ((uint32_t)(quarter * 32) << 16) + buf * acc_stride;
            #pragma unroll 1
            for (int c = first_chunk; c < kBN / kW; c += kChunkStep) {
                const int n0 = tn * kBN + c * kW;
                if (n0 >= p.N) break;                              // warp-uniform: no columns left in this tile
                float res_cur[kW];
                if constexpr (with_res) {                          // the next chunk's values travel while this one is processed
                    #pragma unroll
                    for (int j = 0; j < kW; j++) res_cur[j] = res_next[j];
                    if (n0 + kW * kChunkStep < p.N && c + kChunkStep < kBN / kW) fetch_residual(c + kChunkStep, res_next);
                }
                uint32_t r[kW];
                umma::tmem_load_chunk<kW>(t_row + (uint32_t)(c * kW), r);
                umma::tmem_load_wait();
                {
                    float v[kW];
                    if constexpr (MODE == kModeConv) {                 // no per-row term here; column scales read four at a time
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) {
                            float4 s4 = make_float4(alpha, alpha, alpha, alpha);
                            if (p.fs.b_per_column) s4 = *(const float4*)(my_scale + c * kW + j);
                            v[j] = __fmul_rn(s4.x, __uint_as_float(r[j]));         v[j + 1] = __fmul_rn(s4.y, __uint_as_float(r[j + 1]));
                            v[j + 2] = __fmul_rn(s4.z, __uint_as_float(r[j + 2])); v[j + 3] = __fmul_rn(s4.w, __uint_as_float(r[j + 3]));
                        }
                    } else {
                        #pragma unroll
                        for (int j = 0; j < kW; j++) {
                            const float scale = p.fs.b_per_column ? my_scale[c * kW + j] : alpha;
                            v[j] = __fadd_rn(__fmul_rn(scale, __uint_as_float(r[j])), row_bias);
                        }
                    }
                    if (p.bias.mode == kBiasPerColumn) {
                        #pragma unroll
                        for (int j = 0; j < kW; j += 4) {
                            const float4 b4 = *(const float4*)(my_bias + c * kW + j);
                            v[j] = __fadd_rn(v[j], b4.x); v[j + 1] = __fadd_rn(v[j + 1], b4.y);
                            v[j + 2] = __fadd_rn(v[j + 2], b4.z); v[j + 3] = __fadd_rn(v[j + 3], b4.w);
                        }
                    } else if (p.bias.mode == kBiasMatrix && m < p.M) {
                        float cv[kW];
                        if (p.bias.dtype == DTYPE_FLOAT32) {            // independent loads, issued back to back
                            #pragma unroll
                            for (int j = 0; j < kW; j++) {
                                const long long ci = (n0 + j < p.N) ? bias_index(p.bias, m, n0 + j) : -1;
                                cv[j] = ci >= 0 ? __ldg((const float*)p.bias.ptr + ci) : 0.0f;
                            }
                        } else {
                            #pragma unroll
                            for (int j = 0; j < kW; j++) {
                                const long long ci = (n0 + j < p.N) ? bias_index(p.bias, m, n0 + j) : -1;
                                cv[j] = ci >= 0 ? (float)load_f64_rt(p.bias.ptr, p.bias.dtype, (size_t)ci) : 0.0f;
                            }
                        }
                        #pragma unroll
                        for (int j = 0; j < kW; j++) v[j] = __fmaf_rn(p.beta, cv[j], v[j]);
                    }
                    // levels alone: Relu is part of the clamp below (a negative value quantises to a level <= 0, and 0 lies inside
                    // [lo - z, hi - z]), one instruction per value less
                    const bool relu_in_clamp = MODE == kModeConv && (EPI & kEpiLevels) != 0 && !with_res && p.relu && p.Y == nullptr;
                    if (p.relu && !with_res && !relu_in_clamp) {
                        #pragma unroll
                        for (int j = 0; j < kW; j++) v[j] = fmaxf(v[j], 0.0f);      // same results as v > 0 ? v : 0, NaN and -0 included
                    }
                    if constexpr (MODE == kModeConv) {
                        // NCHW output: for one output channel, consecutive lanes (consecutive padded
                        // positions) are consecutive pixels, so each store instruction is contiguous.
                        if (conv_row) {
                            const size_t base = conv_base + (size_t)(c * kW) * plane_out;
                            if constexpr (with_res) {                  // Add(conv, residual) [-> Relu], as separate float32 operators would round
                                #pragma unroll
                                for (int j = 0; j < kW; j++) {
                                    v[j] = __fadd_rn(v[j], res_cur[j]);
                                    if (p.relu) v[j] = fmaxf(v[j], 0.0f);
                                }
                            }
                            if constexpr ((EPI & kEpiLevels) != 0) {
                                uint16_t* zdst = levels_row + c * kW;          // levels for the next convolution
                                const float ls = lv_scale, linv = lv_inv, zf = lv_zero;
                                // eight values at a time on the fast path without branches (their dependency chains
                                // interleave); a group in which the fast rounding could not decide some value -- a tie
                                // closer than 2^-22 |q|, which also catches |q| >= 2^21 and NaN -- is redone with the
                                // reference's double division
                                const float lo = p.lv.zero_signed ? -128.0f : 0.0f, hi = p.lv.zero_signed ? 127.0f : 255.0f;
                                const float lo_z = relu_in_clamp ? fmaxf(__fsub_rn(lo, zf), 0.0f) : __fsub_rn(lo, zf), hi_z = __fsub_rn(hi, zf);
                                uint32_t packed[kW / 2];
                                #pragma unroll
                                for (int j0 = 0; j0 < kW; j0 += 8) {
                                    float level[8];
                                    bool decided = true;
                                    #pragma unroll
                                    for (int e = 0; e < 8; e++) {
                                        const float q = __fmul_rn(v[j0 + e], linv);
                                        const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                                        decided = decided & (fmaf(fabsf(q), kLevelsTieMargin, fabsf(__fsub_rn(q, rq))) < 0.5f);
                                        level[e] = fminf(fmaxf(rq, lo_z), hi_z);              // clamp(rq + z, lo, hi) - z, all small integers
                                    }
                                    if (!decided) {                     // rare: redo only the values the fast rounding could not decide
                                        #pragma unroll
                                        for (int e = 0; e < 8; e++) {
                                            const float q = __fmul_rn(v[j0 + e], linv);
                                            const float rq = __fsub_rn(__fadd_rn(q, 12582912.0f), 12582912.0f);
                                            if (!(fmaf(fabsf(q), kLevelsTieMargin, fabsf(__fsub_rn(q, rq))) < 0.5f))
                                                level[e] = quantize_level_exact(relu_in_clamp ? fmaxf(v[j0 + e], 0.0f) : v[j0 + e], ls, zf, p.lv.zero_signed);
                                        }
                                    }
                                    #pragma unroll
                                    for (int e = 0; e < 8; e += 2)
                                        packed[(j0 + e) >> 1] = __byte_perm(__float_as_uint(level[e]), __float_as_uint(level[e + 1]), 0x7632);
                                }
                                if (n0 + kW <= p.N && kW == 16 && ((p.lv.Cz | p.lv.C) & 15) == 0) {
                                    // kW contiguous channels of this pixel = one 32-byte sector, written by ONE instruction: two
                                    // 16-byte stores per lane would leave every sector half-written between them
                                    umma::store_global_32B(zdst, packed);
                                } else if (n0 + kW <= p.N) {
                                    #pragma unroll
                                    for (int q4 = 0; q4 < kW / 8; q4++)
                                        *reinterpret_cast<uint4*>(zdst + 8 * q4) = make_uint4(packed[4 * q4], packed[4 * q4 + 1], packed[4 * q4 + 2], packed[4 * q4 + 3]);
                                } else {
                                    #pragma unroll
                                    for (int j = 0; j < kW; j++) if (n0 + j < p.N) zdst[j] = (uint16_t)(packed[j >> 1] >> ((j & 1) * 16));
                                }
                            }
                            if (p.Y == nullptr) {
                                // levels only
                            } else if (p.y_cl) {                       // float32, channels-last: kW consecutive floats of this row
                                float* dst = (float*)p.Y + cl_base + c * kW;
                                if (n0 + kW <= p.N && (p.N & 3) == 0) {
                                    #pragma unroll
                                    for (int j = 0; j < kW; j += 4) *(float4*)(dst + j) = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                } else {
                                    #pragma unroll
                                    for (int j = 0; j < kW; j++) if (n0 + j < p.N) dst[j] = v[j];
                                }
                            } else if (p.dy == DTYPE_FLOAT32) {
                                float* dst = (float*)p.Y + base;
                                #pragma unroll
                                for (int j = 0; j < kW; j++) if (n0 + j < p.N) dst[(size_t)j * plane_out] = v[j];
                            } else if (p.dy == DTYPE_BFLOAT16) {
                                uint16_t* dst = (uint16_t*)p.Y + base;
                                #pragma unroll
                                for (int j = 0; j < kW; j++) if (n0 + j < p.N) dst[(size_t)j * plane_out] = encode_bf16(v[j]);
                            } else {
                                uint16_t* dst = (uint16_t*)p.Y + base;
                                #pragma unroll
                                for (int j = 0; j < kW; j++) if (n0 + j < p.N) dst[(size_t)j * plane_out] = encode_f16(v[j]);
                            }
                        }
                    }
                    if constexpr (MODE != kModeConv) {
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
                    } else if (dtype_bytes(p.dy) == 1) {
                        // 8-bit outputs: QuantizeLinear when a result scale was given, a plain store otherwise.  All of it
                        // stays on the float32 / integer pipes (the float64 pipe is narrow and this runs once per element):
                        // integers through a saturating pack -- NaN, Inf and |q| >= 2^63 become the most negative value
                        // first, as the reference's float -> int64 conversion makes them -- and integer-valued float8
                        // results through the paired hardware convert, which agrees with the reference's encoder on them.
                        #pragma unroll
                        for (int j = 0; j < 32; j += 4) {
                            float q[4];
                            #pragma unroll
                            for (int e = 0; e < 4; e++) {
                                q[e] = v[j + e];
                                if (p.fs.y_scale) q[e] = rintf(__fmul_rn(q[e], y_inv));
                            }
                            uint32_t word = 0;
                            if (p.dy == DTYPE_INT8 || p.dy == DTYPE_UINT8) {
                                int iv[4];
                                #pragma unroll
                                for (int e = 0; e < 4; e++) iv[e] = fabsf(q[e]) < 9.2e18f ? __float2int_rn(q[e]) : (int)0x80000000;
                                word = p.dy == DTYPE_INT8 ? pack_sat_s8x4(iv[0], iv[1], iv[2], iv[3]) : pack_sat_u8x4(iv[0], iv[1], iv[2], iv[3]);
                            } else if (p.fs.y_scale && p.dy == DTYPE_FLOAT8_E4M3) {
                                const uint32_t lo2 = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E4M3);
                                const uint32_t hi2 = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E4M3);
                                word = lo2 | (hi2 << 16);
                            } else if (p.fs.y_scale && p.dy == DTYPE_FLOAT8_E5M2) {
                                const uint32_t lo2 = __nv_cvt_float2_to_fp8x2(make_float2(q[0], q[1]), __NV_SATFINITE, __NV_E5M2);
                                const uint32_t hi2 = __nv_cvt_float2_to_fp8x2(make_float2(q[2], q[3]), __NV_SATFINITE, __NV_E5M2);
                                word = lo2 | (hi2 << 16);
                                #pragma unroll
                                for (int e = 0; e < 4; e++)          // the reference overflows to infinity where the hardware saturates
                                    if (fabsf(q[e]) >= 61440.0f) word = (word & ~(0xFFu << (8 * e))) | ((q[e] < 0.0f ? 0xFCu : 0x7Cu) << (8 * e));
                            } else {
                                #pragma unroll
                                for (int e = 0; e < 4; e++)
                                    word |= (uint32_t)(p.dy == DTYPE_FLOAT8_E4M3 ? encode_e4m3(q[e]) : encode_e5m2(q[e])) << (8 * e);
                            }
                            my_rows[j >> 2] = word;
                        }
                    } else {
                        #pragma unroll
                        for (int j = 0; j < 32; j += 8)
                            *(uint4*)(my_rows + (j >> 1)) = make_uint4(encode_f16x2(v[j], v[j + 1]), encode_f16x2(v[j + 2], v[j + 3]),
                                                                        encode_f16x2(v[j + 4], v[j + 5]), encode_f16x2(v[j + 6], v[j + 7]));
                    }
                    __syncwarp();
                    const int esize = dtype_bytes(p.dy);
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
                        char* dst = (char*)p.Y + (((size_t)bt * p.M + mr) * p.N + n) * esize;
                        if (p.vec_store && n + elems_per_piece <= p.N) {
                            __stcs((uint4*)dst, val);
                        } else {
                            const uint32_t w[4] = {val.x, val.y, val.z, val.w};
                            for (int e = 0; e < elems_per_piece && n + e < p.N; e++) {
                                if (esize == 4) ((uint32_t*)dst)[e] = w[e];
                                else if (esize == 2) ((uint16_t*)dst)[e] = (uint16_t)(w[e >> 1] >> ((e & 1) * 16));
                                else ((uint8_t*)dst)[e] = (uint8_t)(w[e >> 2] >> ((e & 3) * 8));
                            }
                        }
                    }
                    __syncwarp();
                    }
                }
            }
            umma::fence_before_sync();
            __syncwarp();
            if (lane == 0) umma::mbar_arrive(&acc_empty[buf]);
        }
        }   // not the row-linear epilogue
    }

    umma::fence_before_sync();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
    if (warp == 1) {
        umma::fence_after_sync();
        umma::tmem_dealloc(tmem_base, 512);
    }
}


void count_tensor_core_launch();

}  // namespace tops
