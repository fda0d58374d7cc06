// Device-side exhaustive check of the small-float encoders: every float32 bit pattern is encoded
// by the production encoder (hardware convert + fix-ups) and by the bit-level restatement of the
// reference encoder; disagreements are counted.  NaN inputs are skipped for bfloat16 only where
// both produce a NaN code.
#include "common.cuh"
#include "umma.cuh"

namespace tops {

template <int DT>
__global__ void encoder_selftest_kernel(unsigned long long* mismatches, uint32_t first_hi) {
    // each launch covers 2^28 patterns: the top 4 bits come from first_hi
    const uint32_t lo = blockIdx.x * blockDim.x + threadIdx.x;           // 2^20 threads
    unsigned long long bad = 0;
    for (uint32_t k = 0; k < 256; k++) {
        const uint32_t bits = (first_hi << 28) | (k << 20) | lo;
        const float f = __uint_as_float(bits);
        uint32_t fast, slow;
        if constexpr (DT == DTYPE_FLOAT16)          { fast = encode_f16(f);  slow = encode_f16_bits(f); }
        else if constexpr (DT == DTYPE_FLOAT8_E4M3) { fast = encode_e4m3(f); slow = encode_e4m3_bits(f); }
        else if constexpr (DT == DTYPE_FLOAT8_E5M2) { fast = encode_e5m2(f); slow = encode_e5m2_bits(f); }
        else {
            // bfloat16: compare against the hardware convert for non-NaN inputs
            fast = encode_bf16(f);
            slow = (f == f) ? (uint32_t)__bfloat16_as_ushort(__float2bfloat16_rn(f)) : fast;
        }
        bad += (fast != slow);
    }
    if (bad) atomicAdd(mismatches, bad);
}

// One thread waits, with a short clock budget, on a barrier that nothing ever arms: the wait must give up, raise the
// abort flag and return, and the kernel must report through the status word -- the path every tensor-core kernel of
// the library takes when one of its waits expires.  Nothing here spins without a limit.
__global__ void wait_timeout_selftest_kernel(int* status, long long budget_cycles, int* gave_up) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        umma::mbar_init(&bar, 1);
        abort_flag = 0;
        umma::mbar_fence_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const bool done = umma::mbar_wait(&bar, 0, &abort_flag, budget_cycles);
        *gave_up = done ? 0 : 1;
    }
    __syncthreads();
    if (threadIdx.x == 0 && abort_flag && status) atomicExch(status, 1);
}

}  // namespace tops

using namespace tops;

TOPS_API int tops_selftest_wait_timeout(int budget_microseconds) {
    if (!acquire_device()) return -1;
    if (budget_microseconds < 1 || budget_microseconds > 100000) { set_error(TOPS_ERR_INVALID, "tops_selftest_wait_timeout: budget outside 1 .. 100000 us"); return -1; }
    int* gave_up = nullptr;
    if (!TOPS_CUDA_OK(cudaMalloc(&gave_up, sizeof(int)))) return -1;
    cudaStream_t s = current_stream();
    cudaMemsetAsync(gave_up, 0, sizeof(int), s);
    wait_timeout_selftest_kernel<<<1, 32, 0, s>>>(device_status_word(), (long long)budget_microseconds * 2000, gave_up);     // about 2 cycles per ns
    int host = 0;
    const bool ok = TOPS_CHECK_LAUNCH("tops_selftest_wait_timeout") &&
                    TOPS_CUDA_OK(cudaMemcpyAsync(&host, gave_up, sizeof(host), cudaMemcpyDeviceToHost, s)) &&
                    TOPS_CUDA_OK(cudaStreamSynchronize(s));
    cudaFree(gave_up);
    return ok ? host : -1;
}

TOPS_API long long tops_selftest_encoder(DataType dtype) {
    if (!acquire_device()) return -1;
    unsigned long long* counter = nullptr;
    if (!TOPS_CUDA_OK(cudaMalloc(&counter, sizeof(*counter)))) return -1;
    cudaStream_t s = current_stream();
    cudaMemsetAsync(counter, 0, sizeof(*counter), s);
    for (uint32_t hi = 0; hi < 16; hi++) {
        switch ((int)dtype) {
            case DTYPE_FLOAT16:     encoder_selftest_kernel<DTYPE_FLOAT16><<<4096, 256, 0, s>>>(counter, hi); break;
            case DTYPE_BFLOAT16:    encoder_selftest_kernel<DTYPE_BFLOAT16><<<4096, 256, 0, s>>>(counter, hi); break;
            case DTYPE_FLOAT8_E4M3: encoder_selftest_kernel<DTYPE_FLOAT8_E4M3><<<4096, 256, 0, s>>>(counter, hi); break;
            case DTYPE_FLOAT8_E5M2: encoder_selftest_kernel<DTYPE_FLOAT8_E5M2><<<4096, 256, 0, s>>>(counter, hi); break;
            default: cudaFree(counter); set_error(TOPS_ERR_INVALID, "tops_selftest_encoder: not a small float dtype"); return -1;
        }
    }
    unsigned long long host = 0;
    const bool ok = TOPS_CHECK_LAUNCH("tops_selftest_encoder") &&
                    TOPS_CUDA_OK(cudaMemcpyAsync(&host, counter, sizeof(host), cudaMemcpyDeviceToHost, s)) &&
                    TOPS_CUDA_OK(cudaStreamSynchronize(s));
    cudaFree(counter);
    return ok ? (long long)host : -1;
}
