// Conv2d on tensor cores: implicit GEMM as a sum of shifted GEMMs (tensor_ops.c:1036-1114).
//
// Covered: group 1, stride 1, any dilation and padding; X and W both fp16, both bf16, or both fp8;
// output fp32 / bf16 / fp16; C a multiple of 16 bytes of elements.  Everything else takes the
// exact kernel in conv.cu.
//
// 1. X (NCHW) is copied once into a zero-padded channels-last scratch tensor Xp[N][Hp][Wp][C]
//    (top / left padding as given, enough rows / columns at the bottom / right for every tap).
//    Seen as a matrix [N*Hp*Wp, C] its row q = (n, oh, ow) is the top-left input pixel of output
//    (n, oh, ow), and the pixel under filter tap (kh, kw) is simply row q + kh*dil_h*Wp + kw*dil_w.
// 2. W [M][C][KH][KW] is copied into tap-major scratch Wt[KH*KW][M][C].
// 3. The persistent tcgen05 kernel (tc_kernel.cuh) runs one GEMM whose K loop walks the taps: for
//    tap t and channel block cb it TMA-loads 128 rows of Xp starting at tile_row + shift(t) and 256
//    rows of Wt[t], and accumulates into the same tensor-memory tile.  The epilogue adds the bias
//    and scatters the valid rows (oh < OH, ow < OW) into the NCHW output.
// Both scratch tensors come from the stream-ordered pool and go back to it right after the launch.
// Algorithmic flops: 2 * N*OH*OW * M * C*KH*KW; the padded formulation computes (Hp*Wp)/(OH*OW)
// times as many rows (1.07x for 56x56, k3, p1).
#include "conv_common.cuh"
#include "tc_kernel.cuh"

namespace tops {

// NCHW -> zero-padded NHWC.  One CTA handles 64 channels x 64 consecutive padded columns of one
// padded row; elements move as raw bits (ES bytes each).
template <typename E>
__global__ void __launch_bounds__(256) nchw_to_padded_nhwc(const E* __restrict__ x, E* __restrict__ xp,
                                                            int C, int H, int W, int Hp, int Wp, int pt, int pl) {
    constexpr int kVec = 16 / (int)sizeof(E);               // channels per 16-byte store
    constexpr int kPitch = 64 + kVec;                       // tile row pitch in elements (keeps rows 16-byte aligned)
    __shared__ __align__(16) E tile[64][kPitch];            // [column][channel]
    const int wp0 = blockIdx.y * 64, hp = blockIdx.x % Hp, n = blockIdx.x / Hp, c0 = blockIdx.z * 64;
    const int h = hp - pt;
    const bool row_inside = h >= 0 && h < H;
    // read: each thread owns one column and walks 16 channels; a warp reads 32 consecutive
    // columns of one channel plane (contiguous in NCHW); the 16 loads are independent
    {
        const int ww = threadIdx.x & 63, cc0 = threadIdx.x >> 6;
        const int w = wp0 + ww - pl;
        const bool col_inside = row_inside && w >= 0 && w < W;
        const size_t plane = (size_t)H * W;
        const E* src = x + ((size_t)n * C + (size_t)(c0 + cc0)) * plane + (size_t)(row_inside ? h : 0) * W + (col_inside ? w : 0);
        E v[16];
        #pragma unroll
        for (int i = 0; i < 16; i++) {
            const int cc = cc0 + 4 * i;
            v[i] = (col_inside && c0 + cc < C) ? src[(size_t)(4 * i) * plane] : E(0);
        }
        #pragma unroll
        for (int i = 0; i < 16; i++) tile[ww][cc0 + 4 * i] = v[i];
    }
    __syncthreads();
    // write: 16 bytes (kVec channels) per thread, consecutive threads along the channels of one
    // padded position (contiguous in NHWC)
    constexpr int kLanesPerPos = 64 / kVec, kPosPerPass = 256 / kLanesPerPos;
    const int part = threadIdx.x % kLanesPerPos, pos0 = threadIdx.x / kLanesPerPos;
    const int c = c0 + part * kVec;
    if (c < C) {
        #pragma unroll
        for (int pass = 0; pass < 64 / kPosPerPass; pass++) {
            const int ww = pos0 + pass * kPosPerPass, wp = wp0 + ww;
            if (wp < Wp) {
                const uint4 val = *reinterpret_cast<const uint4*>(&tile[ww][part * kVec]);
                *reinterpret_cast<uint4*>(xp + (((size_t)n * Hp + hp) * Wp + wp) * C + c) = val;
            }
        }
    }
}

// The same copy for planes whose byte size is a multiple of 16 (so that every channel plane starts on a 16-byte
// boundary): both sides move 16 bytes per thread.  One CTA takes 64 channels x kTilePos consecutive positions of one
// image plane (flat h * W + w, contiguous in NCHW whatever the width); a thread loads 16 bytes ALONG THE PLANE of four
// channels, the tile is transposed through shared memory, and a thread stores 16 bytes ALONG THE CHANNELS of one
// position.  Only interior cells are written here; zero_padding_cells clears the border.
template <typename E>
__global__ void __launch_bounds__(256) nchw_to_padded_nhwc_vec(const E* __restrict__ x, E* __restrict__ xp,
                                                                int C, int H, int W, int Hp, int Wp, int pt, int pl) {
    constexpr int kVec = 16 / (int)sizeof(E);               // elements per 16 bytes
    constexpr int kTilePos = 16 * kVec;                     // positions per tile: 16 vectors per channel row
    constexpr int kPitchWords = 64 + 1;                     // 256 bytes of payload + one word: rows land on different banks
    __shared__ uint32_t tile[64 * kPitchWords];             // [channel][position], 4-byte granules
    const int plane = H * W;
    const int p0 = blockIdx.x * kTilePos, n = blockIdx.y, c0 = blockIdx.z * 64;
    {
        const int v = threadIdx.x & 15, cc0 = threadIdx.x >> 4;
        const int p = p0 + v * kVec;
        uint4 val[4];
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            const int c = c0 + cc0 + 16 * i;
            val[i] = (p < plane && c < C) ? __ldg(reinterpret_cast<const uint4*>(x + ((size_t)n * C + c) * plane + p)) : make_uint4(0, 0, 0, 0);
        }
        #pragma unroll
        for (int i = 0; i < 4; i++) {
            uint32_t* row = tile + (cc0 + 16 * i) * kPitchWords + v * 4;
            row[0] = val[i].x; row[1] = val[i].y; row[2] = val[i].z; row[3] = val[i].w;
        }
    }
    __syncthreads();
    constexpr int kGroups = 64 / kVec;                      // 16-byte channel groups per position
    constexpr int kPosPerPass = 256 / kGroups;
    const int cg = threadIdx.x % kGroups, pos0 = threadIdx.x / kGroups;
    const int c = c0 + cg * kVec;
    if (c >= C) return;
    const E* tile_e = reinterpret_cast<const E*>(tile);
    #pragma unroll
    for (int pass = 0; pass < kTilePos / kPosPerPass; pass++) {
        const int pp = pos0 + pass * kPosPerPass, p = p0 + pp;
        if (p >= plane) continue;
        __align__(16) E out[kVec];
        #pragma unroll
        for (int j = 0; j < kVec; j++) out[j] = tile_e[(size_t)(cg * kVec + j) * (kPitchWords * 4 / sizeof(E)) + pp];
        const int h = p / W, w = p - h * W;
        *reinterpret_cast<uint4*>(xp + (((size_t)n * Hp + h + pt) * Wp + w + pl) * C + c) = *reinterpret_cast<const uint4*>(out);
    }
}

// Clears the cells of a padded channels-last tensor [N][Hp][Wp][C] that lie outside the H x W interior placed at
// (pt, pl): pt rows on top, Hp - pt - H rows at the bottom, and Wp - W cells in each interior row.  One thread per
// 16 bytes (row_bytes = C * element size is a multiple of 16).
__global__ void __launch_bounds__(256) zero_padding_cells(uint4* __restrict__ xp, int row_vecs, int H, int W, int Hp, int Wp, int pt, int pl) {
    const int top = pt * Wp, bottom = (Hp - pt - H) * Wp, side = Wp - W;
    const int cells = top + bottom + H * side;
    const size_t total = (size_t)cells * row_vecs;
    const int n = blockIdx.y;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        int cell = (int)(i / row_vecs);
        const int v = (int)(i - (size_t)cell * row_vecs);
        int hp, wp;
        if (cell < top) { hp = cell / Wp; wp = cell - hp * Wp; }
        else if (cell < top + bottom) { cell -= top; hp = pt + H + cell / Wp; wp = cell % Wp; }
        else { cell -= top + bottom; const int r = cell / side, k = cell - r * side; hp = pt + r; wp = k < pl ? k : W + k; }
        xp[(((size_t)n * Hp + hp) * Wp + wp) * row_vecs + v] = make_uint4(0, 0, 0, 0);
    }
}

// [M][C][KH*KW] -> [KH*KW][M][C]
template <typename E>
__global__ void __launch_bounds__(256) filters_to_tap_major(const E* __restrict__ w, E* __restrict__ wt, int M, int C, int taps) {
    const size_t total = (size_t)M * C * taps;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const size_t r = i / C;
        const int m = (int)(r % M), t = (int)(r / M);
        wt[i] = w[((size_t)m * C + c) * taps + t];
    }
}

// int8 codes [M][C][KH*KW] -> [KH*KW][M][C] as float16 / bfloat16 values (|code| <= 128 is exact in both)
template <bool BF16>
__global__ void __launch_bounds__(256) int8_filters_to_tap_major(const int8_t* __restrict__ w, uint16_t* __restrict__ wt, int M, int C, int taps) {
    const size_t total = (size_t)M * C * taps;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int c = (int)(i % C);
        const size_t r = i / C;
        const int m = (int)(r % M), t = (int)(r / M);
        const float v = (float)w[((size_t)m * C + c) * taps + t];
        wt[i] = BF16 ? encode_bf16(v) : encode_f16(v);
    }
}

static bool fp8_dtype(int dt) { return dt == DTYPE_FLOAT8_E4M3 || dt == DTYPE_FLOAT8_E5M2; }

ConvTcPlan conv_tc_plan(const Tensor* X, const Tensor* W, const Tensor* Y, const ConvGeom& c, bool int8_weights) {
    ConvTcPlan plan{};
    const int dx = (int)X->dtype, dw = (int)W->dtype, dy = (int)Y->dtype;
    plan.fp8 = !int8_weights && fp8_dtype(dx) && fp8_dtype(dw);
    const bool half16 = (dx == DTYPE_FLOAT16 || dx == DTYPE_BFLOAT16) && (int8_weights ? dw == DTYPE_INT8 : dx == dw);
    if (!plan.fp8 && !half16) return plan;
    if (dy != DTYPE_FLOAT32 && dy != DTYPE_BFLOAT16 && dy != DTYPE_FLOAT16) return plan;
    if (c.G != 1 || c.sh != 1 || c.sw != 1 || c.dh < 1 || c.dw < 1 || c.pt < 0 || c.pl < 0) return plan;
    plan.es = plan.fp8 ? 1 : 2;
    if (((size_t)c.C * plan.es) % 16 != 0) return plan;
    plan.Hp = max(c.H + c.pt, c.OH + (c.KH - 1) * c.dh);
    plan.Wp = max(c.W + c.pl, c.OW + (c.KW - 1) * c.dw);
    plan.rows = (size_t)c.N * plan.Hp * plan.Wp;
    if (plan.rows >= 0x7FFFFF00ull) return plan;
    plan.taps = c.KH * c.KW;
    plan.xp_bytes = plan.rows * c.C * plan.es;
    plan.wt_bytes = (size_t)plan.taps * c.M * c.C * plan.es;
    plan.ok = true;
    return plan;
}

// The layout copy of images [n0, n0 + count) of X into the padded channels-last scratch, on `stream`.
static void conv_tc_layout(const Tensor* X, void* xp, const ConvGeom& c, const ConvTcPlan& plan, int n0, int count, cudaStream_t stream) {
    const int es = plan.es, Hp = plan.Hp, Wp = plan.Wp;
    const char* x = (const char*)X->data + (size_t)n0 * c.C * c.H * c.W * es;
    char* dst = (char*)xp + (size_t)n0 * Hp * Wp * c.C * es;
    // planes that start on 16-byte boundaries take the copy that moves 16 bytes per thread on both sides
    const bool vec_copy = ((size_t)c.H * c.W * es) % 16 == 0 && ((uintptr_t)x & 15) == 0 && ((uintptr_t)dst & 15) == 0 && count <= 65535;
    if (vec_copy) {
        const int tile_pos = 16 * (16 / es);
        const dim3 vgrid((c.H * c.W + tile_pos - 1) / tile_pos, count, (c.C + 63) / 64);
        const int row_vecs = c.C * es / 16;
        const int pad_cells = Hp * Wp - c.H * c.W;
        if (pad_cells > 0) {
            const dim3 zgrid((unsigned)(((size_t)pad_cells * row_vecs + 255) / 256), count);
            zero_padding_cells<<<zgrid, 256, 0, stream>>>((uint4*)dst, row_vecs, c.H, c.W, Hp, Wp, c.pt, c.pl);
        }
        if (es == 2) nchw_to_padded_nhwc_vec<uint16_t><<<vgrid, 256, 0, stream>>>((const uint16_t*)x, (uint16_t*)dst, c.C, c.H, c.W, Hp, Wp, c.pt, c.pl);
        else         nchw_to_padded_nhwc_vec<uint8_t><<<vgrid, 256, 0, stream>>>((const uint8_t*)x, (uint8_t*)dst, c.C, c.H, c.W, Hp, Wp, c.pt, c.pl);
        return;
    }
    const dim3 tgrid(count * Hp, (Wp + 63) / 64, (c.C + 63) / 64);
    if (es == 2) nchw_to_padded_nhwc<uint16_t><<<tgrid, 256, 0, stream>>>((const uint16_t*)x, (uint16_t*)dst, c.C, c.H, c.W, Hp, Wp, c.pt, c.pl);
    else         nchw_to_padded_nhwc<uint8_t><<<tgrid, 256, 0, stream>>>((const uint8_t*)x, (uint8_t*)dst, c.C, c.H, c.W, Hp, Wp, c.pt, c.pl);
}

bool conv_tc_run(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c, const ConvTcPlan& plan,
                 void* xp, void* wt, int* status, const float* w_scale) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    cudaStream_t s = current_stream();
    const int dx = (int)X->dtype, dw = (int)W->dtype, dy = (int)Y->dtype;
    const int es = plan.es, Hp = plan.Hp, Wp = plan.Wp, taps = plan.taps;
    const bool fp8 = plan.fp8;

    const int wgrid = grid_for((size_t)c.M * c.C * taps, 256, st->sm_count, 4);
    if (es == 2) {
        if (dw == DTYPE_INT8 && dx == DTYPE_BFLOAT16)
            int8_filters_to_tap_major<true><<<wgrid, 256, 0, s>>>((const int8_t*)W->data, (uint16_t*)wt, c.M, c.C, taps);
        else if (dw == DTYPE_INT8)
            int8_filters_to_tap_major<false><<<wgrid, 256, 0, s>>>((const int8_t*)W->data, (uint16_t*)wt, c.M, c.C, taps);
        else
            filters_to_tap_major<uint16_t><<<wgrid, 256, 0, s>>>((const uint16_t*)W->data, (uint16_t*)wt, c.M, c.C, taps);
    } else {
        filters_to_tap_major<uint8_t><<<wgrid, 256, 0, s>>>((const uint8_t*)W->data, (uint8_t*)wt, c.M, c.C, taps);
    }

    ShiftedGemm sg;
    sg.wt = wt; sg.es = es; sg.fp8 = fp8;
    sg.a_format = fp8 ? (dx == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (dx == DTYPE_BFLOAT16 ? 1u : 0u);
    sg.b_format = fp8 ? (dw == DTYPE_FLOAT8_E5M2 ? 1u : 0u) : (dw == DTYPE_INT8 ? sg.a_format : (dw == DTYPE_BFLOAT16 ? 1u : 0u));
    sg.Hp = Hp; sg.Wp = Wp; sg.C = c.C; sg.M = c.M; sg.KH = c.KH; sg.KW = c.KW; sg.dil_h = c.dh; sg.dil_w = c.dw;
    sg.OH = c.OH; sg.OW = c.OW;
    sg.dy = dy;
    sg.bias = (B && B->data) ? B->data : nullptr;
    sg.bias_dtype = sg.bias ? (int)B->dtype : DTYPE_FLOAT32;
    sg.status = status;
    if (w_scale) { sg.fs.b_scale = w_scale; sg.fs.b_per_column = 1; }

    conv_tc_layout(X, xp, c, plan, 0, c.N, s);
    if (!TOPS_CHECK_LAUNCH("conv2d_forward (layout copies)")) return false;
    sg.xp = xp;
    sg.Y = Y->data;
    sg.images = c.N;
    return shifted_gemm_launch(sg);
}

bool shifted_gemm_map_ok(const ShiftedGemm& g) {
    CUtensorMap map_a;
    const uint64_t dims_a[2] = {(uint64_t)g.C, (uint64_t)g.images * g.Hp * g.Wp};
    const uint64_t strides_a[1] = {g.a_row_stride_bytes ? (uint64_t)g.a_row_stride_bytes : (uint64_t)g.C * g.es};
    const uint32_t box_a[2] = {(uint32_t)(kRowBytes / g.es), (uint32_t)kBM};
    return make_tensor_map(&map_a, g.xp, g.es, g.fp8, !g.fp8 && g.a_format == 0u, 2, dims_a, strides_a, box_a, nullptr);
}

// The tensor-core part shared by every convolution path: KH * KW shifted GEMMs over a padded
// channels-last activation tensor and tap-major filters that are already in place.
bool shifted_gemm_launch(const ShiftedGemm& g) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    cudaStream_t s = current_stream();
    const int es = g.es, taps = g.KH * g.KW;
    const size_t rows = (size_t)g.images * g.Hp * g.Wp;
    const int k_step = kRowBytes / es;
    CUtensorMap map_a, map_b;
    const uint64_t dims_a[2] = {(uint64_t)g.C, (uint64_t)rows};
    const uint64_t strides_a[1] = {g.a_row_stride_bytes ? (uint64_t)g.a_row_stride_bytes : (uint64_t)g.C * es};
    const uint32_t box_a[2] = {(uint32_t)k_step, (uint32_t)kBM};
    const uint64_t dims_b[3] = {(uint64_t)g.C, (uint64_t)g.M, (uint64_t)taps};
    const uint64_t strides_b[2] = {(uint64_t)g.C * es, (uint64_t)g.M * g.C * es};
    // With at most one column block of filters the box (and the instruction, below) covers only the rows that
    // exist, rounded up to 16: rows beyond them would be zero-filled by the copy engine at the cost of real rows.
    const int n_cols = g.M <= kBN ? ((g.M + 15) / 16) * 16 : kBN;
    const uint32_t box_b[3] = {(uint32_t)k_step, (uint32_t)n_cols, 1u};
    const bool f16 = !g.fp8 && g.a_format == 0u;
    if (!make_tensor_map(&map_a, g.xp, es, g.fp8, f16, 2, dims_a, strides_a, box_a, nullptr) ||
        !make_tensor_map(&map_b, g.wt, es, g.fp8, f16, 3, dims_b, strides_b, box_b, nullptr))
        return false;

    TcParams p;
    // rows beyond the last valid output position of the last image need no tile
    const size_t last_row = ((size_t)(g.images - 1) * g.Hp + (g.OH - 1)) * g.Wp + g.OW;
    p.M = (int)rows; p.N = g.M;
    p.cv.c_blocks = (g.C + k_step - 1) / k_step;
    p.k_blocks = taps * p.cv.c_blocks;
    p.k_step = k_step;
    p.tiles_m = (int)((last_row + kBM - 1) / kBM);
    p.tiles_n = (g.M + kBN - 1) / kBN;
    p.Y = g.Y; p.dy = g.dy;
    p.alpha = 1.0f; p.beta = 1.0f;
    p.bias.ptr = g.bias;
    p.bias.dtype = g.bias_dtype;
    p.bias.mode = g.bias ? kBiasPerColumn : kBiasNone;
    p.bias.rows = 1; p.bias.cols = g.M;
    p.status = g.status;
    p.vec_store = 0;
    p.cv.Wp = g.Wp; p.cv.plane = g.Hp * g.Wp;
    p.cv.by_plane.set((uint32_t)(g.Hp * g.Wp));
    p.cv.by_Wp.set((uint32_t)g.Wp);
    p.cv.images = g.images; p.cv.OH = g.OH; p.cv.OW = g.OW; p.cv.OC = g.M;
    p.cv.KW = g.KW; p.cv.dil_h = g.dil_h; p.cv.dil_w = g.dil_w;
    p.fs = g.fs;
    p.relu = g.relu;
    p.residual = g.residual;
    p.lv = g.lv;
    p.y_cl = g.y_channels_last;
    p.res_cl = g.residual_channels_last;
    p.stage_tx = (uint32_t)(kTileABytes + n_cols * kRowBytes);
    // accumulator buffers and epilogue groups: always more buffers than groups where tensor memory has the columns
    p.acc_buffers = n_cols <= 64 ? 8 : n_cols <= 128 ? 4 : 2;
    p.epilogue_groups = n_cols <= 64 ? 4 : n_cols <= 128 ? 2 : (getenv("TOPS_ONE_EPILOGUE_GROUP") ? 1 : 2);
    // measurement switches; anything tensor memory (512 columns) or the warp layout cannot hold is ignored
    if (const char* e = getenv("TOPS_ACC_BUFFERS")) {
        const int b = atoi(e);
        if ((b == 2 || b == 4 || b == 8) && b * n_cols <= 512) p.acc_buffers = b;
    }
    if (const char* e = getenv("TOPS_EPILOGUE_GROUPS")) {
        const int gr = atoi(e);
        if (gr == 1 || gr == 2 || gr == 4) p.epilogue_groups = gr;
    }
    if (p.epilogue_groups > p.acc_buffers) p.epilogue_groups = p.acc_buffers;
    const uint32_t idesc = umma::instr_desc(g.a_format, g.b_format, kBM, (uint32_t)n_cols);
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < st->sm_count ? tiles : st->sm_count;
    int epi = (g.residual ? kEpiResidual : 0) | (g.lv.z ? kEpiLevels : 0);
    if (g.fp8 && epi != kEpiPlain) return false;                     // the quantised extras exist for 16-bit operands only
    // Row-linear epilogue: the GEMM row is the output pixel (no padded rows to drop) and every float32 tensor the
    // epilogue touches is channels-last, so residual, output and levels are [rows][M] matrices the copy engine moves.
    EpilogueMaps em{};
    const bool rows_linear = !g.fp8 && taps == 1 && g.Hp == g.OH && g.Wp == g.OW && (g.M % 16) == 0 && g.M <= kRowsMaxChannels &&
        (g.Y != nullptr || g.lv.z != nullptr) && (g.Y == nullptr || (g.y_channels_last && g.dy == DTYPE_FLOAT32)) &&
        (g.residual == nullptr || g.residual_channels_last) && (!g.bias || g.bias_dtype == DTYPE_FLOAT32) &&
        (g.lv.z == nullptr || (g.lv.S == 1 && g.lv.pt == 0 && g.lv.pl == 0 && g.lv.Hz == g.OH && g.lv.Wz == g.OW && g.lv.Cz == g.M)) &&
        !getenv("TOPS_NO_ROW_EPILOGUE");
    if (rows_linear) {
        bool maps_ok = true;
        if (g.Y) maps_ok = maps_ok && make_row_box_map(&em.y, g.Y, 4, rows, (uint64_t)g.M, 32, 16);
        if (g.residual) maps_ok = maps_ok && make_row_box_map(&em.res, g.residual, 4, rows, (uint64_t)g.M, 32, 16);
        if (g.lv.z) maps_ok = maps_ok && make_row_box_map(&em.lv, g.lv.z, 2, rows, (uint64_t)g.M, 32, 16);
        if (maps_ok) epi |= kEpiRows;
    }
    // a narrow filter box leaves room for more, smaller pipeline stages in the shared memory the variant reserves
    {
        const uint32_t bytes = (uint32_t)(kTileABytes + n_cols * kRowBytes);
        const int room = tc_stages(kModeConv, epi) * kStageBytes;
        // At most 128 output channels: the multiplies of a K block take less time than the barrier round trip of the two
        // single-thread roles, so two K blocks travel per stage.
        const int per_stage = (n_cols <= 128 && p.k_blocks >= 2 && !getenv("TOPS_ONE_K_BLOCK_PER_STAGE")) ? 2 : 1;
        int st = room / ((int)bytes * per_stage);
        if (st > 8) st = 8;
        if (n_cols < kBN && !getenv("TOPS_FIXED_STAGES")) { p.stages = st; p.stage_bytes = bytes * (uint32_t)per_stage; p.kb_per_stage = per_stage; }
    }
    // programmatic stream serialisation: the kernel waits for its predecessor itself (first statement); TOPS_PDL=0 switches it off
    static const bool pdl = [] { const char* e = getenv("TOPS_PDL"); return !(e && e[0] == '0'); }();
    cudaLaunchAttribute pdl_attr[1];
    pdl_attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    pdl_attr[0].val.programmaticStreamSerializationAllowed = 1;
#define TOPS_CONV_LAUNCH(F8, E)                                                                                              \
    do {                                                                                                                     \
        static_assert(tc_smem_bytes(kModeConv, E) <= 227 * 1024, "the variant's shared memory exceeds what a CTA can have");    \
        if (!ensure_dynamic_smem((const void*)tc_kernel<F8, kModeConv, E>, tc_smem_bytes(kModeConv, E))) return false;          \
        cudaLaunchConfig_t cfg = {};                                                                                         \
        cfg.gridDim = dim3(grid); cfg.blockDim = dim3(tc_threads(kModeConv, E)); cfg.dynamicSmemBytes = tc_smem_bytes(kModeConv, E); \
        cfg.stream = s; cfg.attrs = pdl_attr; cfg.numAttrs = pdl ? 1 : 0;                                                    \
        check_cuda(cudaLaunchKernelEx(&cfg, tc_kernel<F8, kModeConv, E>, map_a, map_b, p, idesc, em), "conv2d_forward (tensor cores)"); \
    } while (0)
    if (g.fp8) TOPS_CONV_LAUNCH(true, kEpiPlain);
    else if (epi == kEpiPlain) TOPS_CONV_LAUNCH(false, kEpiPlain);
    else if (epi == kEpiResidual) TOPS_CONV_LAUNCH(false, kEpiResidual);
    else if (epi == kEpiLevels) TOPS_CONV_LAUNCH(false, kEpiLevels);
    else if (epi == (kEpiResidual | kEpiLevels)) TOPS_CONV_LAUNCH(false, kEpiResidual | kEpiLevels);
    else if (epi == kEpiRows) TOPS_CONV_LAUNCH(false, kEpiRows);
    else if (epi == (kEpiRows | kEpiResidual)) TOPS_CONV_LAUNCH(false, kEpiRows | kEpiResidual);
    else if (epi == (kEpiRows | kEpiLevels)) TOPS_CONV_LAUNCH(false, kEpiRows | kEpiLevels);
    else TOPS_CONV_LAUNCH(false, kEpiRows | kEpiResidual | kEpiLevels);
#undef TOPS_CONV_LAUNCH
    if (!TOPS_CHECK_LAUNCH("conv2d_forward (tensor cores)")) return false;
    count_tensor_core_launch();
    return true;
}

bool conv_tensor_core(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, const ConvGeom& c) {
    if (getenv("TOPS_DISABLE_TC")) return false;
    if ((size_t)c.N * c.OH * c.OW * c.M < (size_t)1 << 16) return false;     // tiny problems: not worth two copies
    const ConvTcPlan plan = conv_tc_plan(X, W, Y, c);
    if (!plan.ok) return false;
    if (!acquire_device()) return true;
    cudaStream_t s = current_stream();
    void *xp = nullptr, *wt = nullptr;
    if (cudaMallocAsync(&xp, plan.xp_bytes, s) != cudaSuccess) { cudaGetLastError(); return false; }
    if (cudaMallocAsync(&wt, plan.wt_bytes, s) != cudaSuccess) { cudaGetLastError(); cudaFreeAsync(xp, s); return false; }
    const bool ok = conv_tc_run(X, W, B, Y, c, plan, xp, wt, device_status_word());
    cudaFreeAsync(xp, s);
    cudaFreeAsync(wt, s);
    return ok;            // false: the exact kernel computes the result instead
}

}  // namespace tops
