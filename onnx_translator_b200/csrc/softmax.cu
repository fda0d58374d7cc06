// Softmax along one axis (tensor_ops.c:1231-1270).  The tensor is viewed as [outer, inner, rem];
// each (outer, rem) pair is an independent row of `inner` elements with element stride `rem`.
//
//   rem == 1, inner <= 1024 : one warp per row, the row lives in registers, max and sum by
//                             warp shuffles.
//   rem == 1, inner  > 1024 : one CTA per row, the decoded row staged in shared memory.
//   rem  > 1 (or any other) : one thread per row walking it with stride `rem` (neighbouring
//                             threads touch neighbouring addresses), in the reference's own
//                             sequential order.
// Arithmetic is double throughout, as in the reference; the parallel variants only change the
// order of the additions inside the sum (results agree to the last float32 bit or one ulp).
#include "common.cuh"

#include <cfloat>

namespace tops {

template <int DT> __device__ __forceinline__ double sm_load(const void* p, int rt, size_t i) {
    if constexpr (DT < 0) return load_f64_rt(p, rt, i);
    else return to_f64<DT>(((const typename Storage<DT>::type*)p)[i]);
}
template <int DT> __device__ __forceinline__ void sm_store(void* p, int rt, size_t i, double v) {
    if constexpr (DT < 0) store_f64_rt(p, rt, i, v);
    else ((typename Storage<DT>::type*)p)[i] = from_f64<DT>(v);
}

__device__ __forceinline__ double warp_max(double v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmax(v, __shfl_xor_sync(0xFFFFFFFFu, v, o));
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
    #pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xFFFFFFFFu, v, o);
    return v;
}

// NaN handling follows the strict '>' scan of the reference: NaN never becomes the maximum.
__device__ __forceinline__ double max_step(double best, double v) { return v > best ? v : best; }

constexpr int kWarpRowMax = 1024;
constexpr int kWarpRowPerLane = kWarpRowMax / 32;

template <int DX, int DO>
__global__ void __launch_bounds__(256) softmax_warp_rows(const void* __restrict__ x, void* __restrict__ y,
                                                          int dx, int dout, uint32_t rows, uint32_t inner) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warps_per_grid = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps_per_grid) {
        const size_t base = (size_t)row * inner;
        double v[kWarpRowPerLane];
        double top = -DBL_MAX;
        #pragma unroll
        for (int k = 0; k < kWarpRowPerLane; k++) {
            const uint32_t j = lane + 32u * k;
            if (j < inner) { v[k] = sm_load<DX>(x, dx, base + j); top = max_step(top, v[k]); }
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = max_step(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
        double total = 0.0;
        #pragma unroll
        for (int k = 0; k < kWarpRowPerLane; k++) {
            const uint32_t j = lane + 32u * k;
            if (j < inner) { v[k] = exp(v[k] - top); total += v[k]; }
        }
        total = warp_sum(total);
        #pragma unroll
        for (int k = 0; k < kWarpRowPerLane; k++) {
            const uint32_t j = lane + 32u * k;
            if (j < inner) sm_store<DO>(y, dout, base + j, v[k] / total);
        }
    }
}

template <int DX, int DO>
__global__ void __launch_bounds__(512) softmax_block_rows(const void* __restrict__ x, void* __restrict__ y,
                                                           int dx, int dout, uint32_t rows, uint32_t inner, int staged) {
    extern __shared__ double row_buf[];
    __shared__ double red[16];
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
    for (uint32_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const size_t base = (size_t)row * inner;
        double top = -DBL_MAX;
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double v = sm_load<DX>(x, dx, base + j);
            if (staged) row_buf[j] = v;
            top = max_step(top, v);
        }
        #pragma unroll
        for (int o = 16; o > 0; o >>= 1) top = max_step(top, __shfl_xor_sync(0xFFFFFFFFu, top, o));
        if (lane == 0) red[warp] = top;
        __syncthreads();
        top = -DBL_MAX;
        for (uint32_t w = 0; w < nwarps; w++) top = max_step(top, red[w]);
        __syncthreads();
        double total = 0.0;
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double e = exp((staged ? row_buf[j] : sm_load<DX>(x, dx, base + j)) - top);
            if (staged) row_buf[j] = e;
            total += e;
        }
        total = warp_sum(total);
        if (lane == 0) red[warp] = total;
        __syncthreads();
        total = 0.0;
        for (uint32_t w = 0; w < nwarps; w++) total += red[w];
        for (uint32_t j = threadIdx.x; j < inner; j += blockDim.x) {
            const double e = staged ? row_buf[j] : exp(sm_load<DX>(x, dx, base + j) - top);
            sm_store<DO>(y, dout, base + j, e / total);
        }
        __syncthreads();
    }
}

template <int DX, int DO>
__global__ void __launch_bounds__(256) softmax_strided_rows(const void* __restrict__ x, void* __restrict__ y,
                                                             int dx, int dout, uint32_t outer, uint32_t inner, uint32_t rem) {
    const size_t rows = (size_t)outer * rem;
    for (size_t r = (size_t)blockIdx.x * blockDim.x + threadIdx.x; r < rows; r += (size_t)gridDim.x * blockDim.x) {
        const size_t o = r / rem, k = r - o * rem;
        const size_t base = o * inner * rem + k;
        double top = -DBL_MAX;
        for (uint32_t j = 0; j < inner; j++) top = max_step(top, sm_load<DX>(x, dx, base + (size_t)j * rem));
        double total = 0.0;
        for (uint32_t j = 0; j < inner; j++) total += exp(sm_load<DX>(x, dx, base + (size_t)j * rem) - top);
        for (uint32_t j = 0; j < inner; j++) {
            const size_t idx = base + (size_t)j * rem;
            sm_store<DO>(y, dout, idx, exp(sm_load<DX>(x, dx, idx) - top) / total);
        }
    }
}

template <int DX, int DO>
static void softmax_launch(const Tensor* x, Tensor* y, uint32_t outer, uint32_t inner, uint32_t rem, DeviceState* st) {
    cudaStream_t s = current_stream();
    const int dx = (int)x->dtype, dout = (int)y->dtype;
    if (rem == 1 && inner <= kWarpRowMax && inner >= 16) {
        const int grid = grid_for((size_t)outer * 32, 256, st->sm_count, 8);
        softmax_warp_rows<DX, DO><<<grid, 256, 0, s>>>(x->data, y->data, dx, dout, outer, inner);
    } else if (rem == 1 && inner > kWarpRowMax) {
        const size_t need = (size_t)inner * sizeof(double);
        const int staged = need <= 200 * 1024;
        if (staged) cudaFuncSetAttribute(softmax_block_rows<DX, DO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)need);
        const int grid = (int)((outer < (uint32_t)st->sm_count * 2) ? outer : (uint32_t)st->sm_count * 2);
        softmax_block_rows<DX, DO><<<grid, 512, staged ? need : 0, s>>>(x->data, y->data, dx, dout, outer, inner, staged);
    } else {
        const int grid = grid_for((size_t)outer * rem, 256, st->sm_count, 8);
        softmax_strided_rows<DX, DO><<<grid, 256, 0, s>>>(x->data, y->data, dx, dout, outer, inner, rem);
    }
    TOPS_CHECK_LAUNCH("softmax_forward");
}

}  // namespace tops

using namespace tops;

TOPS_API void softmax_forward(const Tensor* input, Tensor* output, int axis) {
    if (!input || !output || !input->data || !output->data || input->size != output->size || input->ndim < 1) {
        set_error(TOPS_ERR_INVALID, "softmax_forward: null tensor, size mismatch or rank 0");
        zero_fill(output);
        return;
    }
    if (axis < 0) axis += input->ndim;
    if (axis < 0 || axis >= input->ndim) { set_error(TOPS_ERR_INVALID, "softmax_forward: axis out of range"); zero_fill(output); return; }
    DeviceState* st = acquire_device();
    if (!st || input->size == 0) return;
    size_t outer = 1, rem = 1;
    const size_t inner = (size_t)input->shape[axis];
    for (int d = 0; d < axis; d++) outer *= (size_t)input->shape[d];
    for (int d = axis + 1; d < input->ndim; d++) rem *= (size_t)input->shape[d];
    if (outer > 0x7FFFFFFFull || inner > 0x7FFFFFFFull || rem > 0x7FFFFFFFull) {
        set_error(TOPS_ERR_UNSUPPORTED, "softmax_forward: a dimension exceeds 2^31");
        return;
    }
    const int dx = (int)input->dtype, dout = (int)output->dtype;
    if (dx == DTYPE_FLOAT32 && dout == DTYPE_FLOAT32)        softmax_launch<DTYPE_FLOAT32, DTYPE_FLOAT32>(input, output, outer, inner, rem, st);
    else if (dx == DTYPE_FLOAT16 && dout == DTYPE_FLOAT16)   softmax_launch<DTYPE_FLOAT16, DTYPE_FLOAT16>(input, output, outer, inner, rem, st);
    else if (dx == DTYPE_BFLOAT16 && dout == DTYPE_BFLOAT16) softmax_launch<DTYPE_BFLOAT16, DTYPE_BFLOAT16>(input, output, outer, inner, rem, st);
    else                                                     softmax_launch<-1, -1>(input, output, outer, inner, rem, st);
    finish_op();
}
