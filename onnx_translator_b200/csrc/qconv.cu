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
            // this thread's 16 values (8 channel pairs) first, so that all loads are in flight together
            float v[16];
            #pragma unroll
            for (int i = 0; i < 8; i++) {
                #pragma unroll
                for (int e = 0; e < 2; e++) {
                    const int c = c0 + 2 * (cq + 4 * i) + e;
                    float value = 0.0f;
                    if (c < g.C) {
                        const size_t at = ((size_t)n * g.C + c) * (size_t)plane + (size_t)p;
                        if (XK == 0) value = __ldg((const float*)x + at);
                        else { const uint8_t code = ((const uint8_t*)x)[at]; value = (float)(SIGNED ? (int)(int8_t)code : (int)code); }
                    }
                    v[2 * i + e] = value;
                }
            }
            const float zf = (float)zero;
            float scale = 1.0f, inv = 1.0f;
            if (XK == 0) { scale = __ldg(scale_ptr); inv = __fdividef(1.0f, scale); }
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
        const int h = p / g.W, w = p - h * g.W;
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

// int8 filter codes [M][C][KH][KW] -> bfloat16 levels [KHz*KWz][M][Cz] in the channel order of the activations
__global__ void __launch_bounds__(256) filter_codes_to_levels(const int8_t* __restrict__ w, uint16_t* __restrict__ wt, QGeom g) {
    const size_t total = (size_t)g.KHz * g.KWz * g.M * g.Cz;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
        const int cz = (int)(i % g.Cz);
        const size_t t1 = i / g.Cz;
        const int m = (int)(t1 % g.M), tap = (int)(t1 / g.M);
        const int ta = tap / g.KWz, tb = tap - ta * g.KWz;
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

// x_is_float: X holds float32 values that are quantised on the way (codes of the type of x_zero, int8 when absent)
static int qconv_run(const char* name, const Tensor* X, bool x_is_float, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                     const Tensor* w_scale, const Tensor* B, const Tensor* residual, Tensor* Y, ConvParams* params, int relu) {
    ConvGeom c;
    if (!conv_geometry(name, X, Wq, B, Y, params, &c)) return tops_last_error();
    const bool zero_given = x_zero && x_zero->data;
    const int code_dt = x_is_float ? (zero_given ? (int)x_zero->dtype : DTYPE_INT8) : (int)X->dtype;
    const bool x_ok = (code_dt == DTYPE_INT8 || code_dt == DTYPE_UINT8) && (!x_is_float || X->dtype == DTYPE_FLOAT32);
    if (!x_ok || Wq->dtype != DTYPE_INT8 || !x_scale || !x_scale->data || x_scale->dtype != DTYPE_FLOAT32 || x_scale->size != 1 ||
        !w_scale || !w_scale->data || w_scale->dtype != DTYPE_FLOAT32 || w_scale->size != (size_t)c.M ||
        (zero_given && ((int)x_zero->dtype != code_dt || x_zero->size != 1)) || (B && B->data && B->dtype != DTYPE_FLOAT32) ||
        (residual && residual->data && (residual->dtype != DTYPE_FLOAT32 || residual->size != Y->size))) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: wants int8 / uint8 activation codes (or float32 values) with one float32 scale and one zero point "
                                        "of the code type, int8 filter codes with one float32 scale per output channel, a float32 bias, a float32 residual of Y's size", name);
        zero_fill(Y);
        return tops_last_error();
    }
    const int dy = (int)Y->dtype;
    const bool strided = c.sh == 2 && c.sw == 2 && c.dh == 1 && c.dw == 1;
    if (c.G != 1 || !((c.sh == 1 && c.sw == 1) || strided) || c.dh < 1 || c.dw < 1 || c.pt < 0 || c.pl < 0 ||
        (dy != DTYPE_FLOAT32 && dy != DTYPE_BFLOAT16 && dy != DTYPE_FLOAT16) || (size_t)c.H * c.W >= 0x7FFFFFFFull || c.N > 65535) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: covers group 1, stride 1 (any dilation) or stride 2 (dilation 1), float32 / bfloat16 / float16 output", name);
        zero_fill(Y);
        return tops_last_error();
    }
    if (Y->size == 0) return TOPS_OK;

    QGeom g;
    g.C = c.C; g.H = c.H; g.W = c.W; g.S = c.sh; g.pt = c.pt; g.pl = c.pl; g.M = c.M; g.KH = c.KH; g.KW = c.KW;
    g.KHz = strided ? (c.KH + 1) / 2 : c.KH;
    g.KWz = strided ? (c.KW + 1) / 2 : c.KW;
    const int dil_h = strided ? 1 : c.dh, dil_w = strided ? 1 : c.dw;
    const int need_h = c.OH + (g.KHz - 1) * dil_h, need_w = c.OW + (g.KWz - 1) * dil_w;       // rows / columns the taps reach
    const int have_h = strided ? (c.H + c.pt + 1) / 2 : c.H + c.pt, have_w = strided ? (c.W + c.pl + 1) / 2 : c.W + c.pl;
    g.Hz = need_h > have_h ? need_h : have_h;
    g.Wz = need_w > have_w ? need_w : have_w;
    g.Cz = (g.S * g.S * c.C + 7) & ~7;
    const size_t rows = (size_t)c.N * g.Hz * g.Wz;
    if (rows >= 0x7FFFFF00ull) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: more than 2^31 padded positions", name);
        zero_fill(Y);
        return tops_last_error();
    }
    DeviceState* st = acquire_device();
    if (!st) return tops_last_error();
    cudaStream_t s = current_stream();
    const size_t z_bytes = rows * g.Cz * 2, wt_bytes = (size_t)g.KHz * g.KWz * c.M * g.Cz * 2;
    void *z = nullptr, *wt = nullptr;
    if (cudaMallocAsync(&z, z_bytes, s) != cudaSuccess) { cudaGetLastError(); set_error(TOPS_ERR_OOM, "%s: scratch", name); return tops_last_error(); }
    if (cudaMallocAsync(&wt, wt_bytes, s) != cudaSuccess) {
        cudaGetLastError();
        cudaFreeAsync(z, s);
        set_error(TOPS_ERR_OOM, "%s: scratch", name);
        return tops_last_error();
    }
    // padding cells and padding channels are zero; a 1x1 convolution without padding over a channel
    // count that is a multiple of 8 has neither
    const bool every_cell_written = g.S == 1 && g.Hz == c.H && g.Wz == c.W && g.Cz == c.C;
    bool ok = every_cell_written || TOPS_CUDA_OK(cudaMemsetAsync(z, 0, z_bytes, s));
    const dim3 grid((c.H * c.W + 63) / 64, c.N, (c.C + 63) / 64);
    const void* zero_ptr = zero_given ? x_zero->data : nullptr;
    const float* scale_ptr = (const float*)x_scale->data;
    const bool is_signed = code_dt == DTYPE_INT8;
    if (x_is_float) {
        if (is_signed) activations_to_levels<0, true><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
        else           activations_to_levels<0, false><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
    } else {
        if (is_signed) activations_to_levels<1, true><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
        else           activations_to_levels<1, false><<<grid, 256, 0, s>>>(X->data, (uint16_t*)z, g, scale_ptr, zero_ptr);
    }
    filter_codes_to_levels<<<grid_for(wt_bytes / 2, 256, st->sm_count, 4), 256, 0, s>>>((const int8_t*)Wq->data, (uint16_t*)wt, g);
    ok = ok && TOPS_CHECK_LAUNCH(name);
    if (ok) {
        ShiftedGemm sg;
        sg.xp = z; sg.wt = wt; sg.es = 2; sg.fp8 = false; sg.a_format = 1u; sg.b_format = 1u;
        sg.images = c.N; sg.Hp = g.Hz; sg.Wp = g.Wz; sg.C = g.Cz; sg.M = c.M;
        sg.KH = g.KHz; sg.KW = g.KWz; sg.dil_h = dil_h; sg.dil_w = dil_w; sg.OH = c.OH; sg.OW = c.OW;
        sg.Y = Y->data; sg.dy = dy;
        sg.bias = (B && B->data) ? B->data : nullptr;
        sg.bias_dtype = DTYPE_FLOAT32;
        sg.status = device_status_word();
        sg.fs.a_scale = scale_ptr;
        sg.fs.b_scale = (const float*)w_scale->data;
        sg.fs.b_per_column = 1;
        sg.relu = relu ? 1 : 0;
        sg.residual = (residual && residual->data) ? (const float*)residual->data : nullptr;
        ok = shifted_gemm_launch(sg);
    }
    cudaFreeAsync(z, s);
    cudaFreeAsync(wt, s);
    if (!ok) return tops_last_error();
    finish_op();
    return TOPS_OK;
}

TOPS_API int tops_qlinear_conv_forward(const Tensor* Xq, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                                       const Tensor* w_scale, const Tensor* B, const Tensor* residual, Tensor* Y,
                                       ConvParams* params, int relu) {
    return qconv_run("tops_qlinear_conv_forward", Xq, false, x_scale, x_zero, Wq, w_scale, B, residual, Y, params, relu);
}

TOPS_API int tops_qdq_conv_forward(const Tensor* X, const Tensor* x_scale, const Tensor* x_zero, const Tensor* Wq,
                                   const Tensor* w_scale, const Tensor* B, const Tensor* residual, Tensor* Y,
                                   ConvParams* params, int relu) {
    return qconv_run("tops_qdq_conv_forward", X, true, x_scale, x_zero, Wq, w_scale, B, residual, Y, params, relu);
}
