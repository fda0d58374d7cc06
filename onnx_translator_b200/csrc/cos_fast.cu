// Table cosine at memory speed for float32 / float16 / bfloat16 tensors (tensor_ops.c:815-854).
//
// Same arithmetic as the reference, step for step in double, arranged for the GPU:
//   * the 4097-entry table sits in shared memory as 4096 (lut[k], lut[k+1]) pairs, so the two
//     interpolation operands arrive with one 16-byte shared load;
//   * float -> double is done with integer operations (inputs below 2^-126 behave like 0, which
//     cannot change the rounded result: the interpolation weight would be below 1e-38);
//   * |x| < 4 pi needs no fmod (one exact subtraction at most);
//   * the division by 2 pi is a multiplication by the correctly rounded reciprocal followed by one
//     fused remainder correction, which yields the correctly rounded quotient (Markstein); the
//     exhaustive self-test below compares the whole result with the divide-based formulation for
//     every float32 bit pattern;
//   * floor() comes from a round-down add of 2^52 instead of float <-> int conversions.
#include "elementwise.cuh"

namespace tops {

constexpr double kCosPi = 3.141592653589793238462643383279502884197;
constexpr double kCosTwoPi = 2.0 * kCosPi;
constexpr double kCosCell = kCosTwoPi / 4096.0;        // exact: a power-of-two scaling of 2 pi
constexpr double kCosInvCell = 4096.0 / kCosTwoPi;     // correctly rounded reciprocal of the cell width
constexpr int kCosThreads = 512;
constexpr int kCosCtasPerSm = 3;                       // 3 x 64 KB of shared memory per SM

__device__ __forceinline__ double f32_to_f64_bits(uint32_t mag) {       // mag: |x| as float bits, finite
    if (mag < 0x00800000u) return 0.0;
    return __hiloint2double((int)((mag >> 3) + 0x38000000u), (int)(mag << 29));
}

// Reference formulation, kept for the self-test and for inputs at or above 4 pi.
__device__ __forceinline__ double cos_cell_position_by_division(double r) {
    return __ddiv_rn(__dmul_rn(r, 4096.0), kCosTwoPi);
}
__device__ __forceinline__ double cos_cell_position_fast(double r) {
    const double q0 = __dmul_rn(r, kCosInvCell);
    const double rem = fma(-q0, kCosCell, r);
    return fma(rem, kCosInvCell, q0);
}

template <bool FAST_DIVISION>
__device__ __forceinline__ double cos_from_pairs(uint32_t xbits, const double2* __restrict__ pairs) {
    const uint32_t mag = xbits & 0x7FFFFFFFu;
    if (mag >= 0x7F800000u) return __longlong_as_double(0x7FF8000000000000ll);   // undefined upstream
    const double ax = f32_to_f64_bits(mag);
    double r;
    if (ax < kCosTwoPi) r = ax;
    else if (ax < 2.0 * kCosTwoPi) r = __dsub_rn(ax, kCosTwoPi);          // exact, equals fmod
    else r = fmod(ax, kCosTwoPi);
    const double pos = FAST_DIVISION ? cos_cell_position_fast(r) : cos_cell_position_by_division(r);
    const double shifted = __dadd_rd(pos, 4503599627370496.0);             // 2^52 + floor(pos)
    int k = __double2loint(shifted);
    double w = __dsub_rn(pos, __dsub_rn(shifted, 4503599627370496.0));
    if (k >= 4096) { k = 4095; w = 0.0; }
    const double2 p = pairs[k];
    return __dadd_rn(__dmul_rn(p.x, __dsub_rn(1.0, w)), __dmul_rn(p.y, w));
}

__device__ __forceinline__ void load_cos_pairs(double2* pairs, const double* __restrict__ lut) {
    for (int k = threadIdx.x; k < 4096; k += blockDim.x) pairs[k] = make_double2(lut[k], lut[k + 1]);
    __syncthreads();
}

template <int DT>
__global__ void __launch_bounds__(kCosThreads, kCosCtasPerSm)
cos_fast_kernel(const typename Storage<DT>::type* __restrict__ x, typename Storage<DT>::type* __restrict__ y,
                const double* __restrict__ lut, size_t n, int vec_ok) {
    extern __shared__ double2 cos_pairs[];
    load_cos_pairs(cos_pairs, lut);
    using S = typename Storage<DT>::type;
    constexpr int V = 16 / (int)sizeof(S);
    const size_t runs = (n + V - 1) / V;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += (size_t)gridDim.x * blockDim.x) {
        const size_t i0 = r * V;
        const uint32_t nv = (uint32_t)((n - i0) < (size_t)V ? (n - i0) : (size_t)V);
        Run<S, V> in, out;
        if (vec_ok && nv == V) load_bytes_stream<16>(x + i0, &in);
        else for (int j = 0; j < V; j++) in.v[j] = (uint32_t)j < nv ? x[i0 + j] : S(0);
        float f[V];
        #pragma unroll
        for (int j = 0; j < V; j++) f[j] = __double2float_rn(cos_from_pairs<true>(__float_as_uint(to_f32<DT>(in.v[j])), cos_pairs));
        encode_floats<DT, V>(f, out);
        if (vec_ok && nv == V) store_bytes_stream<16>(y + i0, &out);
        else for (int j = 0; j < V; j++) if ((uint32_t)j < nv) y[i0 + j] = out.v[j];
    }
}

// Exhaustive: every finite float32 input, fast formulation against the divide-based one.
__global__ void __launch_bounds__(kCosThreads, kCosCtasPerSm)
cos_selftest_kernel(const double* __restrict__ lut, unsigned long long* mismatches, uint32_t hi4) {
    extern __shared__ double2 cos_pairs[];
    load_cos_pairs(cos_pairs, lut);
    unsigned long long bad = 0;
    const uint32_t lanes = gridDim.x * blockDim.x;                 // must divide 2^28
    for (uint32_t low = blockIdx.x * blockDim.x + threadIdx.x; low < (1u << 28); low += lanes) {
        const uint32_t bits = (hi4 << 28) | low;
        if ((bits & 0x7FFFFFFFu) >= 0x7F800000u) continue;
        const double a = cos_from_pairs<true>(bits, cos_pairs), b = cos_from_pairs<false>(bits, cos_pairs);
        bad += (__double_as_longlong(a) != __double_as_longlong(b));
    }
    if (bad) atomicAdd(mismatches, bad);
}

// Returns true when it launched the fast kernel (same-dtype float32 / float16 / bfloat16).
bool cos_fast(const Tensor* x, Tensor* y, const double* lut) {
    const int dt = (int)x->dtype;
    if (dt != (int)y->dtype || (dt != DTYPE_FLOAT32 && dt != DTYPE_FLOAT16 && dt != DTYPE_BFLOAT16)) return false;
    DeviceState* st = acquire_device();
    if (!st) return true;
    const int smem = 4096 * (int)sizeof(double2);
    cudaStream_t s = current_stream();
    const void* kernel = dt == DTYPE_FLOAT32 ? (const void*)cos_fast_kernel<DTYPE_FLOAT32>
                       : dt == DTYPE_FLOAT16 ? (const void*)cos_fast_kernel<DTYPE_FLOAT16> : (const void*)cos_fast_kernel<DTYPE_BFLOAT16>;
    if (!ensure_dynamic_smem(kernel, (size_t)smem)) return false;    // the general kernel computes the result; the error stays recorded
    if (x->size == 0) return true;
    const int vec_ok = aligned_to(x->data, 16) && aligned_to(y->data, 16);
    const int V = 16 / dtype_bytes(dt);
    const size_t runs = (x->size + V - 1) / V;
    const int grid = grid_for(runs, kCosThreads, st->sm_count, kCosCtasPerSm);
    if (dt == DTYPE_FLOAT32)      cos_fast_kernel<DTYPE_FLOAT32><<<grid, kCosThreads, smem, s>>>((const float*)x->data, (float*)y->data, lut, x->size, vec_ok);
    else if (dt == DTYPE_FLOAT16) cos_fast_kernel<DTYPE_FLOAT16><<<grid, kCosThreads, smem, s>>>((const uint16_t*)x->data, (uint16_t*)y->data, lut, x->size, vec_ok);
    else                          cos_fast_kernel<DTYPE_BFLOAT16><<<grid, kCosThreads, smem, s>>>((const uint16_t*)x->data, (uint16_t*)y->data, lut, x->size, vec_ok);
    TOPS_CHECK_LAUNCH("cos_forward");
    return true;
}

}  // namespace tops

using namespace tops;

TOPS_API long long tops_selftest_cos(void) {
    DeviceState* st = acquire_device();
    const double* lut = cos_lut_device();
    if (!st || !lut) return -1;
    if (!ensure_dynamic_smem((const void*)cos_selftest_kernel, 4096 * sizeof(double2))) return -1;
    unsigned long long* counter = nullptr;
    if (!TOPS_CUDA_OK(cudaMalloc(&counter, sizeof(*counter)))) return -1;
    cudaStream_t s = current_stream();
    cudaMemsetAsync(counter, 0, sizeof(*counter), s);
    for (uint32_t hi = 0; hi < 16; hi++)
        cos_selftest_kernel<<<256, kCosThreads, 4096 * sizeof(double2), s>>>(lut, counter, hi);
    unsigned long long host = 0;
    const bool ok = TOPS_CHECK_LAUNCH("tops_selftest_cos") &&
                    TOPS_CUDA_OK(cudaMemcpyAsync(&host, counter, sizeof(host), cudaMemcpyDeviceToHost, s)) &&
                    TOPS_CUDA_OK(cudaStreamSynchronize(s));
    cudaFree(counter);
    return ok ? (long long)host : -1;
}
