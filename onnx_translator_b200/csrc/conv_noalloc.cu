// tops_conv2d_forward_noalloc: the tensor-core convolution with its scratch in a fixed array.
//
// Who this is for.  conv2d_forward borrows two scratch tensors from the CUDA memory pool on every
// call (a padded channels-last copy of X and a tap-major copy of W).  Some callers must not let a
// library allocate device memory at all: a serving process that has handed the whole GPU to its
// own arena allocator and accounts for every byte, a caller inside a section where an allocation
// could block on the driver or fail late, a process pinned to a fixed memory budget by its
// operator.  For them this entry point does the same computation with scratch that already
// exists: a file-scope device array that is part of the loaded library image.
//
// Cost of that choice: the array (kScratchBytes, 36 MiB) is part of the library's device image, so
// every GPU on which the library's device code gets loaded holds it until the process exits, whether
// or not this function is ever called there.  (With CUDA's default lazy module loading that happens
// at the first kernel launch or symbol lookup of this library on that GPU -- possibly this call.)
//
// Rules for callers
//   * Size limit: the padded copy of X (N * Hp * Wp * C elements) must fit kInputBytes = 32 MiB and
//     the filter copy (KH * KW * M * C elements) kFilterBytes = 4 MiB.  Larger problems are rejected
//     with TOPS_ERR_UNSUPPORTED and a message that names the sizes; use conv2d_forward for those.
//   * Only the cases the tensor-core path covers are accepted (group 1, stride 1, fp16 / bf16 / fp8
//     inputs of one kind, fp32 / bf16 / fp16 output, C a multiple of 16 bytes); there is no silent
//     switch to another kernel here.
//   * The first call on each device looks up the device address of the array (and, if nothing in
//     the library ran on that device before, creates the library's stream).  Make that first call
//     before starting any stream capture -- or call tops_conv2d_noalloc_prepare() there, which does
//     this set-up and nothing else.
//   * A bounded wait that expires inside the kernel is reported (TOPS_ERR_DEVICE_TIMEOUT at the next
//     tops_sync) through a word of pinned host memory.  This function never allocates it: it exists
//     once tops_conv2d_noalloc_prepare() or any other tensor-core operator of the library has run.
//     Without it an expired wait still ends the kernel, but nothing reports it.
//   * All calls share the one array.  It still holds the previous call's data when the next call
//     starts; every byte a call reads it first writes (padding included), so nothing needs
//     clearing.  Two calls that overlap on the GPU (different streams, or different host threads)
//     race on it: keep calls to this function ordered on one stream.
//   * No cudaMalloc / cudaFree / pool allocation / host allocation happens in here.
#include "conv_common.cuh"

#include <mutex>

namespace tops {

constexpr size_t kInputBytes = (size_t)32 << 20;
constexpr size_t kFilterBytes = (size_t)4 << 20;
constexpr size_t kScratchBytes = kInputBytes + kFilterBytes;

// In host code this name is only a handle for the runtime's symbol table, not a device address:
// the address each device gave the array is fetched once with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char g_conv_scratch[kScratchBytes];

static unsigned char* g_scratch_on_device[kMaxDevices] = {nullptr};
static std::mutex g_scratch_mutex;

// Device address of the scratch array on the CURRENT device (acquire_device made it current).
static unsigned char* scratch_for_current_device() {
    int dev = -1;
    if (!TOPS_CUDA_OK(cudaGetDevice(&dev)) || dev < 0 || dev >= kMaxDevices) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    if (!g_scratch_on_device[dev]) {
        void* ptr = nullptr;
        if (!TOPS_CUDA_OK(cudaGetSymbolAddress(&ptr, g_conv_scratch))) return nullptr;
        g_scratch_on_device[dev] = (unsigned char*)ptr;
    }
    return g_scratch_on_device[dev];
}

}  // namespace tops

using namespace tops;

TOPS_API void tops_conv2d_forward_noalloc(const Tensor* X, const Tensor* W, const Tensor* B, Tensor* Y, ConvParams* params) {
    const char* name = "tops_conv2d_forward_noalloc";
    ConvGeom c;
    if (!conv_geometry(name, X, W, B, Y, params, &c)) return;
    if (Y->size == 0) return;
    const ConvTcPlan plan = conv_tc_plan(X, W, Y, c);
    if (!plan.ok) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: only group 1, stride 1, fp16/bf16/fp8 inputs with fp32/bf16/fp16 output and "
                  "C a multiple of 16 bytes are covered", name);
        zero_fill(Y);
        return;
    }
    if (plan.xp_bytes > kInputBytes || plan.wt_bytes > kFilterBytes) {
        set_error(TOPS_ERR_UNSUPPORTED, "%s: scratch needed (%zu bytes for the padded input, %zu for the filters) exceeds the "
                  "fixed %zu / %zu bytes", name, plan.xp_bytes, plan.wt_bytes, kInputBytes, kFilterBytes);
        zero_fill(Y);
        return;
    }
    if (!acquire_device()) return;                         // no usable device: nothing can be written either
    unsigned char* scratch = scratch_for_current_device();
    if (!scratch) { zero_fill(Y); finish_op(); return; }   // the CUDA error is already recorded
    if (!conv_tc_run(X, W, B, Y, c, plan, scratch, scratch + kInputBytes, device_status_word_if_created())) {
        set_error(TOPS_ERR_CUDA, "%s: the kernels could not be launched", name);      // keeps an earlier, more specific error
        zero_fill(Y);
    }
    finish_op();
}

TOPS_API int tops_conv2d_noalloc_prepare(void) {
    if (!acquire_device()) return tops_last_error();
    if (!scratch_for_current_device()) return tops_last_error();
    (void)device_status_word();                             // pinned host word for time-out reports (allocates once per process)
    return TOPS_OK;
}

TOPS_API size_t tops_conv2d_noalloc_limits(size_t* input_bytes, size_t* filter_bytes) {
    if (input_bytes) *input_bytes = kInputBytes;
    if (filter_bytes) *filter_bytes = kFilterBytes;
    return kScratchBytes;
}
