// Convolution of a quantised graph in one call:
//
//     Y = [Relu]( Conv( DequantizeLinear(Xq, x_scale, x_zero), DequantizeLinear(Wq, w_scale, 0) ) + B [+ R] )
//
// i.e. the chain QuantizeLinear -> DequantizeLinear -> Conv (weights through DequantizeLinear) [-> Relu]
// that wraps every convolution of a QDQ network (reference operators: nn/Operators.py:427-473, 475-548,
// C functions tensor_ops.c:999-1034, 1036-1114), starting from the activation CODES.
//
// The integer levels (code - zero point, |level| <= 255, and the weight codes, |code| <= 128) are
// exact in bfloat16, so they go to the tensor cores as bfloat16 operands; every product is exact and
// the fp32 accumulator only rounds once a partial sum exceeds 2^24.  The scales are applied to the
// accumulator: x_scale * w_scale[m].  The reference multiplies each operand by its scale first
// (rounding each to float32) and accumulates in double: the results differ by the accumulation
// order and by those per-element roundings, the tolerance class of the tensor-core convolution.
//
// tops_qdq_conv_forward starts one step earlier, from the float32 activations: the QuantizeLinear that
// produces the codes is evaluated inside the layout pass (same codes, bit for bit).
//
// Layout work (one pass over the activations, one over the filters):
//   * stride 1: codes NCHW -> levels, zero-padded channels-last [N][Hp][Wp][C8] (C8 = C rounded up to 8);
//   * stride 2: the same with a space-to-depth step, Z[A][B][(r,s,c)] = Xpad[2A + r][2B + s][c], which
//     turns the stride-2 KH x KW convolution into a stride-1 ceil(KH/2) x ceil(KW/2) convolution over
//     4C channels (filter taps that fall outside the original window are zero);
//   * stride 2 with a 1 x 1 filter and no padding only ever reads every second pixel: the layout pass keeps just
//     those (a stride-1 1 x 1 convolution over the subsampled image, C channels instead of 4C);
//   * filters [M][C][KH][KW] -> tap-major [taps][M][C8'] in the same channel order.
// Then the shifted-GEMM tensor-core kernel (conv_tc.cu, tc_kernel.cuh) runs unchanged.
#include "conv_common.cuh"
#include "qdq_math.cuh"

namespace tops {

struct QGeom {
    int C, H, W;           // input
    int S;                 // stride (1 or 2), the same in both directions
    int pt, pl;
    int Hz, Wz, Cz;        // levels tensor: rows, columns, channels (S*S*C rounded up to 8)
    int KH, KW, KHz, KWz;  // original and space-to-depth filter extents
    int M;
    int sub, srcW, src_plane;   // sub = 1: the layout pass reads every second row and column of a srcW-wide source plane
    FastDiv by_W, by_plane, by_groups, by_Wz;   // the layout passes' index arithmetic: W, H * W, ceil(C / 8), Wz (set by set_divisors)
    void set_divisors() { by_W.set((uint32_t)W); by_plane.set((uint32_t)(H * W)); by_groups.set((uint32_t)((C + 7) >> 3)); by_Wz.set((uint32_t)Wz); }
};

__device__ __forceinline__ uint16_t level_bits(int v) {        // small integer -> bfloat16 bits (exact for |v| <= 256)
    return (uint16_t)(__float_as_uint((float)v) >> 16);
}

// Activations -> levels.  One CTA: 64 channels x 64 consecutive positions of one image plane (flat
// h * W + w, so reads are contiguous whatever the plane's width); a shared-memory transpose lets the
// reads run along the NCHW plane and the writes along the channels of the channels-last output.
// Each input element lands in exactly one cell: (A, B) = (h + pt, w + pl) for stride 1, and
// (A, B, r, s) = ((h + pt) / 2, (w + pl) / 2, (h + pt) % 2, (w + pl) % 2) for stride 2.  Padding
// cells and padding channels are not written: the caller clears the tensor first.
// XK 0: float32 values, quantised here exactly as quantize_linear_forward does (SIGNED: int8 codes,
// else uint8); XK 1: 8-bit codes.
template <int XK, bool SIGNED>
__global__ void __launch_bounds__(256) activations_to_levels(const void* __restrict__ x, uint16_t* __restrict__ z, QGeom g,
                                                             const float* __restrict__ scale_ptr, const void* __restrict__ zero_ptr) {
    // [position][channel pair], 33 words per row: conflict-free for the column-wise fill (consecutive
    // lanes = consecutive positions) and for the row-wise drain (8 lanes x 4 words per position)
    __shared__ uint32_t tile[64][33];
    const int plane = g.H * g.W;
    const int p0 = blockIdx.x * 64, n = blockIdx.y, c0 = blockIdx.z * 64;
    int zero = 0;
    if (zero_ptr) zero = SIGNED ? (int)*(const int8_t*)zero_ptr : (int)*(const uint8_t*)zero_ptr;
    {
        const int pp = threadIdx.x & 63, cq = threadIdx.x >> 6;
        const int p = p0 + pp;
        if (p < plane) {
            size_t src_p = (size_t)p;
            if (g.sub) { const int hs = (int)g.by_W.div((uint32_t)p); src_p = (size_t)(2 * hs) * g.srcW + 2 * (p - hs * g.W); }
            // this thread's 16 values (8 channel pairs) first, so that all loads are in flight together
            float v[16];
            const size_t cs = (size_t)g.src_plane;                      // distance between channels
            const size_t first = ((size_t)n * g.C + c0 + 2 * cq) * cs + src_p;    // channel c0 + 2 cq of this position
            if (XK == 0 && c0 + 64 <= g.C) {                             // a full tile of float32 values: one address, constant steps
                const float* src = (const float*)x + first;
                #pragma unroll
                for (int i = 0; i < 8; i++) {
                    v[2 * i] = __ldg(src + (size_t)(8 * i) * cs);
                    v[2 * i + 1] = __ldg(src + (size_t)(8 * i + 1) * cs);
                }
            } else {
                #pragma unroll
                for (int i = 0; i < 8; i++) {
                    #pragma unroll
                    for (int e = 0; e < 2; e++) {
                        const int c = c0 + 2 * (cq + 4 * i) + e;
                        float value = 0.0f;
                        if (c < g.C) {
                            const size_t at = first + (size_t)(8 * i + e) * cs;
                            if (XK == 0) value = __ldg((const float*)x + at);
                            else { const uint8_t code = ((const uint8_t*)x)[at]; value = (float)(SIGNED ? (int)(int8_t)code : (int)code); }
                        }
                        v[2 * i + e] = value;
                    }
                }
            }
            const float zf = (float)zero;
            float scale = 1.0f, inv = 1.0f;
            if (XK == 0) { scale = __ldg(scale_ptr); inv = quantize_reciprocal(scale); }
            #pragma unroll
            for (int i = 0; i < 8; i++) {
                float level[2];
                #pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = c0 + 2 * (cq + 4 * i) + e;
                    if (c >= g.C) level[e] = 0.0f;
                    else if (XK == 0) level[e] = quantize_level_8bit<SIGNED ? DTYPE_INT8 : DTYPE_UINT8>(v[2 * i + e], scale, inv, zf);
                    else level[e] = __fsub_rn(v[2 * i + e], zf);
                }
                // bfloat16 bits of two small integers: the upper halves of their float32 patterns
                tile[pp][cq + 4 * i] = __byte_perm(__float_as_uint(level[0]), __float_as_uint(level[1]), 0x7632);
            }
        }
    }
    __syncthreads();
    const int part = threadIdx.x & 7, pos0 = threadIdx.x >> 3;     // 8 lanes x 8 channels (16 bytes) per position
    const int c = c0 + part * 8;
    if (c >= g.C) return;
    const bool vec = (g.C & 7) == 0;                              // every 8-channel group starts on 16 bytes
    #pragma unroll
    for (int pass = 0; pass < 2; pass++) {
        const int pp = pos0 + pass * 32, p = p0 + pp;
        if (p >= plane) continue;
        const int h = (int)g.by_W.div((uint32_t)p), w = p - h * g.W;
        int A = h + g.pt, B = w + g.pl, slot = 0;
        if (g.S == 2) { slot = ((A & 1) * 2 + (B & 1)) * g.C; A >>= 1; B >>= 1; }
        uint16_t* dst = z + (((size_t)n * g.Hz + A) * g.Wz + B) * g.Cz + slot + c;
        const uint4 val = make_uint4(tile[pp][part * 4], tile[pp][part * 4 + 1], tile[pp][part * 4 + 2], tile[pp][part * 4 + 3]);
        if (vec) {
            *reinterpret_cast<uint4*>(dst) = val;
        } else {
            const uint32_t words[4] = {val.x, val.y, val.z, val.w};
            #pragma unroll
            for (int e = 0; e < 8; e++) if (c + e < g.C) dst[e] = (uint16_t)(words[e >> 1] >> ((e & 1) * 16));
        }
    }
}

// The same for few input channels (C <= 8, e.g. the RGB stem): the 64-channel tiles above would be almost
// empty.  Here a thread owns one CELL of the levels tensor -- for stride 2 the 2 x 2 input positions
// that fold into it, all channels -- and writes it whole, padding channels and cells outside the image
// included (zeros), 16 bytes at a time: every cell is written, so the tensor needs no clearing, and no
// store is narrower than a sector's half.  (One thread per input position wrote its C levels as C
// separate 2-byte stores.)
// CC: the channel count when it is 1, 3 or 4 (the cell's levels then stay in registers), 0 for any other.
template <int XK, bool SIGNED, int CC>
__global__ void __launch_bounds__(256) cells_from_few_channels(const void* __restrict__ x, uint16_t* __restrict__ z, QGeom g,
                                                               const float* __restrict__ scale_ptr, const void* __restrict__ zero_ptr) {
    const int cells = g.Hz * g.Wz, n = blockIdx.y;
    const int q = blockIdx.x * blockDim.x + threadIdx.x;
    if (q >= cells) return;
    int zero = 0;
    if (zero_ptr) zero = SIGNED ? (int)*(const int8_t*)zero_ptr : (int)*(const uint8_t*)zero_ptr;
    const float zf = (float)zero;
    float scale = 1.0f, inv = 1.0f;
    if (XK == 0) { scale = __ldg(scale_ptr); inv = quantize_reciprocal(scale); }
    const int a = (int)g.by_Wz.div((uint32_t)q), b = q - a * g.Wz;
    const size_t plane = (size_t)g.H * g.W;
    const int C = CC ? CC : g.C;
    uint16_t level[32];                                           // S * S * C <= 32 channels of the cell, then the padding
    #pragma unroll
    for (int k = 0; k < 32; k++) level[k] = 0;
    #pragma unroll
    for (int rs = 0; rs < 4; rs++) {
        if (rs >= g.S * g.S) break;
        const int r = g.S == 2 ? rs >> 1 : 0, sx = g.S == 2 ? rs & 1 : 0;
        const int h = g.S * a + r - g.pt, w = g.S * b + sx - g.pl;
        if (h < 0 || h >= g.H || w < 0 || w >= g.W) continue;     // a padding position: its levels stay zero
        const size_t at = (size_t)n * C * plane + (size_t)h * g.W + w;
        #pragma unroll
        for (int c = 0; c < 8; c++) {
            if (c >= C) break;
            float lv;
            if (XK == 0) lv = quantize_level_8bit<SIGNED ? DTYPE_INT8 : DTYPE_UINT8>(__ldg((const float*)x + at + (size_t)c * plane), scale, inv, zf);
            else { const uint8_t code = ((const uint8_t*)x)[at + (size_t)c * plane]; lv = __fsub_rn((float)(SIGNED ? (int)(int8_t)code : (int)code), zf); }
            level[rs * C + c] = (uint16_t)(__float_as_uint(lv) >> 16);
        }
    }
    uint4* dst = (uint4*)(z + ((size_t)n * cells + q) * g.Cz);      // Cz is a multiple of 8: 16-byte pieces
    #pragma unroll
    for (int k = 0; k < 4; k++) {
        if (8 * k >= g.Cz) break;
        dst[k] = make_uint4(level[8 * k] | (uint32_t)level[8 * k + 1] << 16, level[8 * k + 2] | (uint32_t)level[8 * k + 3] << 16,
                            level[8 * k + 4] | (uint32_t)level[8 * k + 5] << 16, level[8 * k + 6] | (uint32_t)level[8 * k + 7] << 16);
    }
}

// The same from a channels-last source [N][H][W][C] (the float32 edges a fused graph keeps between its
// quantised convolutions): source and destination both run along the channels, so there is nothing to
// transpose.  A thread owns eight consecutive channels of one position: 32 bytes in, 16 bytes out.
template <int XK, bool SIGNED>
__global__ void __launch_bounds__(256) channels_last_to_levels(const void* __restrict__ x, uint16_t* __restrict__ z, QGeom g, int images,
                                                               const float* __restrict__ scale_ptr, const void* __restrict__ zero_ptr) {
    const int groups = (g.C + 7) >> 3, plane = g.H * g.W;
    const size_t total = (size_t)images * plane * groups;
    int zero = 0;
    if (zero_ptr) zero = SIGNED ? (int)*(const int8_t*)zero_ptr : (int)*(const uint8_t*)zero_ptr;
    const float zf = (float)zero;
    float scale = 1.0f, inv = 1.0f;
    if (XK == 0) { scale = __ldg(scale_ptr); inv = quantize_reciprocal(scale); }
    const bool vec = (g.C & 7) == 0;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        // (image, position, channel group) of item i: three divisions by run-time values, by multiply-high while i fits
        // 31 bits (positions always do: the caller refuses more than 2^31 of them)
        int cg;
        uint32_t t;
        if (i < 0x80000000ull) { t = g.by_groups.div((uint32_t)i); cg = (int)((uint32_t)i - t * (uint32_t)groups); }
        else { t = (uint32_t)(i / groups); cg = (int)(i - (size_t)t * groups); }
        const int n = (int)g.by_plane.div(t), p = (int)(t - (uint32_t)n * (uint32_t)plane);
        const int h = (int)g.by_W.div((uint32_t)p), w = p - h * g.W;
        size_t src_p = (size_t)p;
        if (g.sub) src_p = (size_t)(2 * h) * g.srcW + 2 * w;
        const size_t at = ((size_t)n * g.src_plane + src_p) * g.C + (size_t)cg * 8;
        float v[8];
        if (XK == 0) {
            if (vec) {
                const float4 a = __ldg((const float4*)((const float*)x + at)), b = __ldg((const float4*)((const float*)x + at + 4));
                v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
            } else {
                #pragma unroll
                for (int e = 0; e < 8; e++) v[e] = cg * 8 + e < g.C ? __ldg((const float*)x + at + e) : 0.0f;
            }
        } else {
            #pragma unroll
            for (int e = 0; e < 8; e++) {
                const uint8_t code = cg * 8 + e < g.C ? ((const uint8_t*)x)[at + e] : (uint8_t)zero;
                v[e] = (float)(SIGNED ? (int)(int8_t)code : (int)code);
            }
        }
        uint32_t packed[4];
        #pragma unroll
        for (int e = 0; e < 8; e += 2) {
            float level[2];
            #pragma unroll
            for (int k = 0; k < 2; k++) {
                if (cg * 8 + e + k >= g.C) level[k] = 0.0f;
                else if (XK == 0) level[k] = quantize_level_8bit<SIGNED ? DTYPE_INT8 : DTYPE_UINT8>(v[e + k], scale, inv, zf);
                else level[k] = __fsub_rn(v[e + k], zf);
            }
            packed[e >> 1] = __byte_perm(__float_as_uint(level[0]), __float_as_uint(level[1]), 0x7632);
        }
        int A = h + g.pt, B = w + g.pl, slot = 0;
        if (g.S == 2) { slot = ((A & 1) * 2 + (B & 1)) * g.C; A >>= 1; B >>= 1; }
        uint16_t* dst = z + (((size_t)n * g.Hz + A) * g.Wz + B) * g.Cz + slot + cg * 8;
        if (vec) {
            *reinterpret_cast<uint4*>(dst) = make_uint4(packed[0], packed[1], packed[2], packed[3]);
        } else {
            #pragma unroll
            for (int e = 0; e < 8; e++) if (cg * 8 + e < g.C) dst[e] = (uint16_t)(packed[e >> 1] >> ((e & 1) * 16));
        }
    }
}

// int8 filter codes [M][C][KH][KW] -> bfloat16 levels in the channel order of the activations:
// [KHz*KWz][M][Cz], or with `merged` [KHz][M][KWz*Cz] (the taps of one filter row side by side, for
// the layout in which one activation row covers KWz neighbouring cells)
__global__ void __launch_bounds__(256) filter_codes_to_levels(const int8_t* __restrict__ w, uint16_t* __restrict__ wt, QGeom g, int merged) {
    const size_t total = (size_t)g.KHz * g.KWz * g.M * g.Cz;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cz = (int)(i % g.Cz);
        const size_t t1 = i / g.Cz;
        int m, ta, tb;
        if (merged) { tb = (int)(t1 % g.KWz); const size_t t2 = t1 / g.KWz; m = (int)(t2 % g.M); ta = (int)(t2 / g.M); }
        else { m = (int)(t1 % g.M); const int tap = (int)(t1 / g.M); ta = tap / g.KWz; tb = tap - ta * g.KWz; }
        int v = 0;
        if (cz < g.S * g.S * g.C) {
            const int rs = cz / g.C, c = cz - rs * g.C;
            const int r = rs / g.S, s = rs - r * g.S;
            const int kh = g.S * ta + r, kw = g.S * tb + s;
            if (kh < g.KH && kw < g.KW) v = w[(((size_t)m * g.C + c) * g.KH + kh) * g.KW + kw];
        }
        wt[i] = level_bits(v);
    }
}

}  // namespace tops

using namespace tops;

namespace tops {

// Geometry of the levels tensor a convolution reads: rows / columns / channels and filter extents
// after the optional space-to-depth step.  False when the fused kernel does not cover the case.
static bool levels_geometry(int C, int H, int W, int M, int KH, int KW, const ConvParams* prm, QGeom* g, int* OH, int* OW,
                            int* dil_h, int* dil_w) {
    if (!prm || !prm->pads || !prm->strides || !prm->dilations || prm->group != 1) return false;
    const int pt = prm->pads[0], pl = prm->pads[1], pb = prm->pads[2], pr = prm->pads[3];
    const int sh = prm->strides[0], sw = prm->strides[1], dh = prm->dilations[0], dw = prm->dilations[1];
    const bool strided = sh == 2 && sw == 2 && dh == 1 && dw == 1;
    if (!((sh == 1 && sw == 1) || strided) || dh < 1 || dw < 1 || pt < 0 || pl < 0 || pb < 0 || pr < 0 || KH < 1 || KW < 1) return false;
    const int eh = H + pt + pb - dh * (KH - 1) - 1, ew = W + pl + pr - dw * (KW - 1) - 1;
    if (eh < 0 || ew < 0) return false;
    *OH = eh / sh + 1;
    *OW = ew / sw + 1;
    g->C = C; g->H = H; g->W = W; g->S = sh; g->pt = pt; g->pl = pl; g->M = M; g->KH = KH; g->KW = KW;
    g->KHz = strided ? (KH + 1) / 2 : KH;
    g->KWz = strided ? (KW + 1) / 2 : KW;
    *dil_h = strided ? 1 : dh;
    *dil_w = strided ? 1 : dw;
    const int need_h = *OH + (g->KHz - 1) * *dil_h, need_w = *OW + (g->KWz - 1) * *dil_w;     // rows / columns the taps reach
    const int have_h = strided ? (H + pt + 1) / 2 : H + pt, have_w = strided ? (W + pl + 1) / 2 : W + pl;
    g->Hz = need_h > have_h ? need_h : have_h;
    g->Wz = need_w > have_w ? need_w : have_w;
    g->Cz = (g->S * g->S * C + 7) & ~7;
    g->sub = 0; g->srcW = W; g->src_plane = H * W;
    return true;
}

static bool one_f32(const Tensor* t) { return t && t->data && t->dtype == DTYPE_FLOAT32 && t->size == 1; }

static int qconv_fail(const char* name, int code, const char* what, Tensor* y) {
    set_error(code, "%s: %s", name, what);
    zero_fill(y);
    return tops_last_error();
}

static int qconv_run(const char* name, const QConvCall& q) {
    const Tensor *X = q.x, *Wq = q.w_codes, *B = q.bias, *R = q.residual;
    Tensor* Y = q.y;
    if (!X || !X->data || !Wq || !Wq->data || Wq->ndim != 4 || X->ndim != 4 || (!Y && !q.y_levels))
        return qconv_fail(name, TOPS_ERR_INVALID, "null argument, or tensors that are not 4-D, or no output given", Y);
    const bool x_cl = !q.x_levels && q.x_channels_last;            // x is [N, H, W, C]
    const int N = q.x_levels ? q.x_shape[0] : X->shape[0], C = q.x_levels ? q.x_shape[1] : X->shape[x_cl ? 3 : 1];
    const int H = q.x_levels ? q.x_shape[2] : X->shape[x_cl ? 1 : 2], W = q.x_levels ? q.x_shape[3] : X->shape[x_cl ? 2 : 3];
    const int M = Wq->shape[0], KH = Wq->shape[2], KW = Wq->shape[3];
    QGeom g;
    int OH, OW, dil_h, dil_w;
    if (N < 1 || N > 65535 || C < 1 || Wq->shape[1] != C || (size_t)H * W >= 0x7FFFFFFFull ||
        !levels_geometry(C, H, W, M, KH, KW, q.params, &g, &OH, &OW, &dil_h, &dil_w))
        return qconv_fail(name, TOPS_ERR_UNSUPPORTED, "covers group 1, stride 1 (any dilation) or stride 2 (dilation 1), W of shape [M, C, KH, KW]", Y);

    if (!q.x_levels && g.S == 2 && KH == 1 && KW == 1 && C > 8 && !q.params->pads[0] && !q.params->pads[1] && !q.params->pads[2] && !q.params->pads[3]) {
        // every second pixel is all this convolution reads: lay out just those, then it is a stride-1 1 x 1 convolution
        g.H = OH; g.W = OW; g.S = 1; g.pt = g.pl = 0; g.Hz = OH; g.Wz = OW; g.Cz = (C + 7) & ~7;
        g.sub = 1; g.srcW = W; g.src_plane = H * W;
    }
    g.set_divisors();
    const bool zero_given = q.x_zero && q.x_zero->data;
    const bool x_is_float = !q.x_levels && X->dtype == DTYPE_FLOAT32;
    const int code_dt = q.x_levels ? DTYPE_INT8 : x_is_float ? (zero_given ? (int)q.x_zero->dtype : DTYPE_INT8) : (int)X->dtype;
    if (q.x_levels) {
        if (X->dtype != DTYPE_BFLOAT16 || X->shape[0] != N || X->shape[1] != g.Hz || X->shape[2] != g.Wz || X->shape[3] != g.Cz)
            return qconv_fail(name, TOPS_ERR_INVALID, "the levels tensor does not have the shape tops_qconv_levels_shape gives for this convolution", Y);
    } else if ((code_dt != DTYPE_INT8 && code_dt != DTYPE_UINT8) || (zero_given && ((int)q.x_zero->dtype != code_dt || q.x_zero->size != 1))) {
        return qconv_fail(name, TOPS_ERR_UNSUPPORTED, "wants float32 values or int8 / uint8 codes, and one zero point of the code type", Y);
    }
    if (Wq->dtype != DTYPE_INT8 || !one_f32(q.x_scale) || !q.w_scale || !q.w_scale->data || q.w_scale->dtype != DTYPE_FLOAT32 ||
        q.w_scale->size != (size_t)M || (B && B->data && (B->dtype != DTYPE_FLOAT32 || B->size < (size_t)M)))
        return qconv_fail(name, TOPS_ERR_UNSUPPORTED, "wants int8 filter codes, one float32 activation scale, one float32 scale per output channel, a float32 bias", Y);
    const size_t out_elems = (size_t)N * M * OH * OW;
    int dy = DTYPE_FLOAT32;
    if (Y && q.y_channels_last) {
        dy = (int)Y->dtype;
        if (!Y->data || Y->ndim != 4 || Y->shape[0] != N || Y->shape[1] != OH || Y->shape[2] != OW || Y->shape[3] != M || dy != DTYPE_FLOAT32)
            return qconv_fail(name, TOPS_ERR_INVALID, "a channels-last Y must be float32 [N, OH, OW, M]", Y);
    } else if (Y) {
        dy = (int)Y->dtype;
        if (!Y->data || Y->ndim != 4 || Y->shape[0] != N || Y->shape[1] != M || Y->shape[2] != OH || Y->shape[3] != OW ||
            (dy != DTYPE_FLOAT32 && dy != DTYPE_BFLOAT16 && dy != DTYPE_FLOAT16))
            return qconv_fail(name, TOPS_ERR_INVALID, "Y must be [N, M, OH, OW] in float32 / bfloat16 / float16", Y);
    }
    if (R && R->data && (R->dtype != DTYPE_FLOAT32 || R->size != out_elems))
        return qconv_fail(name, TOPS_ERR_INVALID, "the residual must be float32 with the output's element count", Y);

    LevelsOut lv;
    if (q.y_levels) {
        QGeom ng;
        int noh, now, ndh, ndw;
        const bool nz = q.next_zero && q.next_zero->data;
        if (!q.y_levels->data || q.y_levels->dtype != DTYPE_BFLOAT16 || q.y_levels->ndim != 4 || !one_f32(q.next_scale) || (M & 7) ||
            (nz && ((q.next_zero->dtype != DTYPE_INT8 && q.next_zero->dtype != DTYPE_UINT8) || q.next_zero->size != 1)) ||
            !levels_geometry(M, OH, OW, 1, q.next_kernel[0], q.next_kernel[1], q.next_params, &ng, &noh, &now, &ndh, &ndw) ||
            q.y_levels->shape[0] != N || q.y_levels->shape[1] != ng.Hz || q.y_levels->shape[2] != ng.Wz || q.y_levels->shape[3] != ng.Cz)
            return qconv_fail(name, TOPS_ERR_INVALID, "levels output: needs a bfloat16 tensor of the shape tops_qconv_levels_shape gives for the next "
                                                     "convolution, its float32 scale (and 8-bit zero point), and an output channel count that is a multiple of 8", Y);
        lv.z = (uint16_t*)q.y_levels->data;
        lv.scale = (const float*)q.next_scale->data;
        lv.zero = nz ? q.next_zero->data : nullptr;
        lv.zero_signed = !nz || q.next_zero->dtype == DTYPE_INT8;
        lv.S = ng.S; lv.pt = ng.pt; lv.pl = ng.pl; lv.Hz = ng.Hz; lv.Wz = ng.Wz; lv.Cz = ng.Cz; lv.C = M;
    }
    if (out_elems == 0) return TOPS_OK;
    const size_t rows = (size_t)N * g.Hz * g.Wz;
    if (rows >= 0x7FFFFF00ull) return qconv_fail(name, TOPS_ERR_UNSUPPORTED, "more than 2^31 padded positions", Y);

    DeviceState* st = acquire_device();
    if (!st) return tops_last_error();
    cudaStream_t s = current_stream();
    const size_t z_bytes = rows * g.Cz * 2, wt_bytes = (size_t)g.KHz * g.KWz * M * g.Cz * 2;
    void *z = nullptr, *wt = nullptr;
    bool ok = true;
    if (q.x_levels) {
        z = X->data;
    } else {
        // 128 bytes of slack: with merged taps the last rows of the activation matrix reach past the last cell
        if (cudaMallocAsync(&z, z_bytes + 128, s) != cudaSuccess) { cudaGetLastError(); return qconv_fail(name, TOPS_ERR_OOM, "scratch", nullptr); }
        // padding cells and padding channels are zero; a 1x1 convolution without padding over a channel
        // count that is a multiple of 8 has neither
        const bool few = !x_cl && C <= 8;                          // the per-cell kernel writes every cell and padding channel itself
        const bool every_cell_written = few || (g.S == 1 && g.Hz == g.H && g.Wz == g.W && g.Cz == C);
        ok = every_cell_written ? (!few || TOPS_CUDA_OK(cudaMemsetAsync((char*)z + z_bytes, 0, 128, s)))
                                : TOPS_CUDA_OK(cudaMemsetAsync(z, 0, z_bytes + 128, s));
        const dim3 grid((H * W + 63) / 64, N, (C + 63) / 64);
        const dim3 grid_few((g.Hz * g.Wz + 255) / 256, N);
        const void* zero_ptr = zero_given ? q.x_zero->data : nullptr;
        const float* scale_ptr = (const float*)q.x_scale->data;
        const bool is_signed = code_dt == DTYPE_INT8;
        if (x_cl) {
            const int cl_grid = grid_for((size_t)N * g.H * g.W * ((C + 7) / 8), 256, st->sm_count, 8);
            if (x_is_float && is_signed)       channels_last_to_levels<0, true><<<cl_grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, N, scale_ptr, zero_ptr);
            else if (x_is_float)               channels_last_to_levels<0, false><<<cl_grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, N, scale_ptr, zero_ptr);
            else if (is_signed)                channels_last_to_levels<1, true><<<cl_grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, N, scale_ptr, zero_ptr);
            else                               channels_last_to_levels<1, false><<<cl_grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, N, scale_ptr, zero_ptr);
        } else if (C <= 8) {
#define TOPS_FEW(XK, SG)                                                                                                        \
            do {                                                                                                                \
                if (C == 1)      cells_from_few_channels<XK, SG, 1><<<grid_few, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr); \
                else if (C == 3) cells_from_few_channels<XK, SG, 3><<<grid_few, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr); \
                else if (C == 4) cells_from_few_channels<XK, SG, 4><<<grid_few, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr); \
                else             cells_from_few_channels<XK, SG, 0><<<grid_few, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr); \
            } while (0)
            if (x_is_float && is_signed) TOPS_FEW(0, true);
            else if (x_is_float)         TOPS_FEW(0, false);
            else if (is_signed)          TOPS_FEW(1, true);
            else                         TOPS_FEW(1, false);
#undef TOPS_FEW
        } else if (x_is_float) {
            if (is_signed) activations_to_levels<0, true><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
            else           activations_to_levels<0, false><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
        } else {
            if (is_signed) activations_to_levels<1, true><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
            else           activations_to_levels<1, false><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
        }
    }
    // The filters in tensor-core layout: scratch of this call, or a tensor kept by the caller between calls
    // (shape [1 + merged][elements], so that a cache made for the other layout is recognised).
    const bool cached = q.filter_cache && *q.filter_cache;
    Tensor* keep = nullptr;
    if (cached) {
        keep = *q.filter_cache;
        if (!keep->data || keep->dtype != DTYPE_BFLOAT16 || keep->ndim != 2 || (size_t)keep->shape[1] != wt_bytes / 2) {
            if (!q.x_levels) cudaFreeAsync(z, s);
            return qconv_fail(name, TOPS_ERR_INVALID, "the filter cache was made for another convolution", Y);
        }
        wt = keep->data;
    } else if (!q.filter_cache) {
        if (cudaMallocAsync(&wt, wt_bytes, s) != cudaSuccess) {
            cudaGetLastError();
            if (!q.x_levels) cudaFreeAsync(z, s);
            return qconv_fail(name, TOPS_ERR_OOM, "scratch", nullptr);
        }
    }
    // Few channels: the KWz taps of a filter row are KWz neighbouring cells, i.e. contiguous memory, so one
    // activation "row" of KWz * Cz channels (rows overlapping, one cell apart) feeds a whole filter row per K
    // block instead of a mostly empty K block per tap.  Only for scratch built here (it has the slack the last
    // rows need) and only if the driver accepts the overlapping map.
    ShiftedGemm sg;
    sg.xp = z; sg.wt = wt; sg.es = 2; sg.fp8 = false; sg.a_format = 1u; sg.b_format = 1u;
    sg.images = N; sg.Hp = g.Hz; sg.Wp = g.Wz; sg.C = g.Cz; sg.M = M;
    sg.KH = g.KHz; sg.KW = g.KWz; sg.dil_h = dil_h; sg.dil_w = dil_w; sg.OH = OH; sg.OW = OW;
    bool merged = false;
    if (!q.x_levels && dil_w == 1 && g.KWz > 1 && g.Cz * g.KWz <= 64) {
        ShiftedGemm trial = sg;
        trial.C = g.Cz * g.KWz; trial.KW = 1; trial.a_row_stride_bytes = g.Cz * 2;
        if (shifted_gemm_map_ok(trial)) { sg = trial; merged = true; }
    }
    if (q.filter_cache && !cached) {
        const int shape[2] = {merged ? 2 : 1, (int)(wt_bytes / 2)};
        keep = wt_bytes / 2 <= 0x3FFFFFFFull ? tops_create_uninit(shape, 2, DTYPE_BFLOAT16) : nullptr;
        if (!keep) {
            if (!q.x_levels) cudaFreeAsync(z, s);
            return qconv_fail(name, TOPS_ERR_OOM, "filter cache", nullptr);
        }
        *q.filter_cache = keep;
        wt = keep->data;
        sg.wt = wt;
    }
    if (cached && (keep->shape[0] == 2) != merged) {
        if (!q.x_levels) cudaFreeAsync(z, s);
        return qconv_fail(name, TOPS_ERR_INVALID, "the filter cache was made for the other filter layout", Y);
    }
    if (!cached) filter_codes_to_levels<<<grid_for(wt_bytes / 2, 256, st->sm_count, 4), 256, 0, s>>>((const int8_t*)Wq->data, (uint16_t*)wt, g, merged ? 1 : 0);
    ok = ok && TOPS_CHECK_LAUNCH(name);
    if (ok) {
        sg.Y = Y ? Y->data : nullptr; sg.dy = dy;
        sg.bias = (B && B->data) ? B->data : nullptr;
        sg.bias_dtype = DTYPE_FLOAT32;
        sg.status = device_status_word();
        sg.fs.a_scale = (const float*)q.x_scale->data;
        sg.fs.b_scale = (const float*)q.w_scale->data;
        sg.fs.b_per_column = 1;
        sg.relu = q.relu ? 1 : 0;
        sg.residual = (R && R->data) ? (const float*)R->data : nullptr;
        sg.lv = lv;
        sg.y_channels_last = (Y && q.y_channels_last) ? 1 : 0;
        sg.residual_channels_last = (sg.residual && q.residual_channels_last) ? 1 : 0;
        ok = shifted_gemm_launch(sg);
    }
    if (!q.x_levels) cudaFreeAsync(z, s);
    if (!q.filter_cache) cudaFreeAsync(wt, s);
    if (!ok) return tops_last_error();
    finish_op();
    return TOPS_OK;
}

}  // namespace tops

TOPS_API int tops_qconv_forward(const QConvCall* call) {
    if (!call) { set_error(TOPS_ERR_INVALID, "tops_qconv_forward: null call"); return tops_last_error(); }
    return qconv_run("tops_qconv_forward", *call);
}

TOPS_API int tops_qconv_levels_shape(const int x_shape[4], const int kernel[2], const ConvParams* params, int levels_shape[4]) {
    QGeom g;
    int oh, ow, dh, dw;
    if (!x_shape || !kernel || !levels_shape || !levels_geometry(x_shape[1], x_shape[2], x_shape[3], 1, kernel[0], kernel[1], params, &g, &oh, &ow, &dh, &dw)) {
        set_error(TOPS_ERR_UNSUPPORTED, "tops_qconv_levels_shape: null argument or a convolution the quantised kernel does not cover");
        return tops_last_error();
    }
    levels_shape[0] = x_shape[0]; levels_shape[1] = g.Hz; levels_shape[2] = g.Wz; levels_shape[3] = g.Cz;
    return TOPS_OK;
}

static QConvCall plain_call(const Tensor* X, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq, const Tensor* w_scale,
                            const Tensor* B, const Tensor* R, Tensor* Y, ConvParams* params, int relu) {
    QConvCall q = {};
    q.x = X; q.x_scale = x_scale; q.x_zero = x_zero; q.w_codes = Wq; q.w_scale = w_scale; q.bias = B; q.residual = R;
    q.params = params; q.relu = relu; q.y = Y;
    return q;
}

TOPS_API int tops_qlinear_conv_forward(const Tensor* Xq, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                                       const Tensor* w_scale, const Tensor* B, const Tensor* residual, Tensor* Y,
                                       ConvParams* params, int relu) {
    if (Xq && Xq->dtype == DTYPE_FLOAT32) {
        set_error(TOPS_ERR_UNSUPPORTED, "tops_qlinear_conv_forward: wants int8 / uint8 codes (tops_qdq_conv_forward takes float32 values)");
        zero_fill(Y);
        return tops_last_error();
    }
    return qconv_run("tops_qlinear_conv_forward", plain_call(Xq, x_scale, x_zero, Wq, w_scale, B, residual, Y, params, relu));
}

TOPS_API int tops_qdq_conv_forward(const Tensor* X, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                                   const Tensor* w_scale, const Tensor* B, const Tensor* residual, Tensor* Y,
                                   ConvParams* params, int relu) {
    if (X && X->dtype != DTYPE_FLOAT32) {
        set_error(TOPS_ERR_UNSUPPORTED, "tops_qdq_conv_forward: wants float32 values (tops_qlinear_conv_forward takes the codes)");
        zero_fill(Y);
        return tops_last_error();
    }
    return qconv_run("tops_qdq_conv_forward", plain_call(X, x_scale, x_zero, Wq, w_scale, B, residual, Y, params, relu));
}
