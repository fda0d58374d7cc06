// Runtime of the operator library: device / stream selection, sticky error state, tensor
// allocation from the stream-ordered pool, views, transfers, the cosine table and the host-side
// broadcast planner.
#include "common.cuh"

#include <atomic>
#include <cstdarg>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <new>

namespace tops {

// ---- errors --------------------------------------------------------------------------------------
static std::atomic<int> g_error{TOPS_OK};
static std::mutex       g_error_mutex;
static char             g_error_message[512] = "";

void set_error(int code, const char* fmt, ...) {
    std::lock_guard<std::mutex> lock(g_error_mutex);
    if (g_error.load() != TOPS_OK) return;          // first error wins
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error_message, sizeof(g_error_message), fmt, ap);
    va_end(ap);
    g_error.store(code);
    if (const char* strict = getenv("TOPS_STRICT")) {
        if (strict[0] == '1') { fprintf(stderr, "tensor_ops_b200: %s\n", g_error_message); abort(); }
    }
}

bool check_cuda(cudaError_t e, const char* what) {
    if (e == cudaSuccess) return true;
    const int code = (e == cudaErrorMemoryAllocation) ? TOPS_ERR_OOM
                   : (e == cudaErrorNoDevice || e == cudaErrorInsufficientDriver) ? TOPS_ERR_NO_DEVICE
                   : TOPS_ERR_CUDA;
    set_error(code, "%s: %s", what, cudaGetErrorString(e));
    return false;
}

// ---- devices and streams ----------------------------------------------------------------------------
static DeviceState   g_devices[kMaxDevices];
static cudaStream_t  g_user_stream[kMaxDevices] = {nullptr};
static bool          g_user_stream_set[kMaxDevices] = {false};
static std::mutex    g_device_mutex;
static std::atomic<int> g_managed{0};
static thread_local int t_device = -1;

static int default_device() {
    static int cached = -2;
    if (cached != -2) return cached;
    int dev = 0;
    if (const char* s = getenv("TOPS_DEVICE")) dev = atoi(s);
    else if (const char* r = getenv("LOCAL_RANK")) dev = atoi(r);
    cached = dev;
    return dev;
}

DeviceState* acquire_device() {
    const int dev = t_device >= 0 ? t_device : default_device();
    if (dev < 0 || dev >= kMaxDevices) { set_error(TOPS_ERR_INVALID, "device index %d out of range", dev); return nullptr; }
    if (!TOPS_CUDA_OK(cudaSetDevice(dev))) return nullptr;
    DeviceState* st = &g_devices[dev];
    if (!st->ready) {
        std::lock_guard<std::mutex> lock(g_device_mutex);
        if (!st->ready) {
            if (!TOPS_CUDA_OK(cudaStreamCreateWithFlags(&st->own_stream, cudaStreamNonBlocking))) return nullptr;
            int sms = 0;
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0) st->sm_count = sms;
            // keep freed blocks cached in the pool instead of returning them to the driver
            cudaMemPool_t pool;
            if (cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
                unsigned long long keep = ~0ull;
                cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep);
            }
            st->ready = true;
        }
    }
    return st;
}

static int current_device_index() { return t_device >= 0 ? t_device : default_device(); }

// (kernel, device) pairs whose dynamic shared-memory limit has been raised.  A flat table under the device
// mutex: a few dozen kernels at most, looked up once per launch.
struct SmemOptIn { const void* kernel; size_t bytes; unsigned device_mask; };
static SmemOptIn g_smem_opt_in[128];
static int       g_smem_opt_in_count = 0;

bool ensure_dynamic_smem(const void* kernel, size_t bytes) {
    const int dev = current_device_index();
    if (dev < 0 || dev >= kMaxDevices) return false;
    std::lock_guard<std::mutex> lock(g_device_mutex);
    SmemOptIn* slot = nullptr;
    for (int i = 0; i < g_smem_opt_in_count; i++)
        if (g_smem_opt_in[i].kernel == kernel && g_smem_opt_in[i].bytes == bytes) { slot = &g_smem_opt_in[i]; break; }
    if (slot && (slot->device_mask >> dev & 1u)) return true;
    if (!TOPS_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes))) return false;
    if (!slot && g_smem_opt_in_count < 128) { slot = &g_smem_opt_in[g_smem_opt_in_count++]; *slot = SmemOptIn{kernel, bytes, 0u}; }
    if (slot) slot->device_mask |= 1u << dev;      // table full: the attribute is simply set again next time
    return true;
}

// Host-only view of that bookkeeping for the tests: how many devices hold the opt-in of entry `index`
// (-1 past the end).
int smem_opt_in_devices(int index) {
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (index < 0 || index >= g_smem_opt_in_count) return -1;
    return __builtin_popcount(g_smem_opt_in[index].device_mask);
}

cudaStream_t current_stream() {
    const int dev = current_device_index();
    if (dev < 0 || dev >= kMaxDevices) return nullptr;
    return g_user_stream_set[dev] ? g_user_stream[dev] : g_devices[dev].own_stream;
}

bool managed_mode() { return g_managed.load() != 0; }

void finish_op() {
    if (managed_mode()) TOPS_CUDA_OK(cudaStreamSynchronize(current_stream()));
}

// ---- tensors ----------------------------------------------------------------------------------------
constexpr uint64_t kTensorMagic = 0x544F50535F423230ull;   // "TOPS_B20"

enum AllocKind { kPool = 0, kManaged = 1, kWrapped = 2, kView = 3 };

struct TensorImpl {
    Tensor           pub;        // first member: Tensor* and TensorImpl* are the same address
    uint64_t         magic;
    std::atomic<int> refs;
    TensorImpl*      base;       // views keep their base alive
    int              device;
    int              kind;
};

static TensorImpl* impl_of(const Tensor* t) {
    if (!t) return nullptr;
    TensorImpl* impl = reinterpret_cast<TensorImpl*>(const_cast<Tensor*>(t));
    return impl->magic == kTensorMagic ? impl : nullptr;
}

static TensorImpl* new_header(const int* shape, int ndim, DataType dtype) {
    if (ndim < 0 || (ndim > 0 && !shape) || !dtype_valid((int)dtype)) {
        set_error(TOPS_ERR_INVALID, "create_tensor: bad shape or dtype %d", (int)dtype);
        return nullptr;
    }
    TensorImpl* impl = new (std::nothrow) TensorImpl();
    if (!impl) { set_error(TOPS_ERR_OOM, "create_tensor: host allocation failed"); return nullptr; }
    impl->pub.shape = (int*)malloc(sizeof(int) * (size_t)(ndim > 0 ? ndim : 1));
    if (!impl->pub.shape) { delete impl; set_error(TOPS_ERR_OOM, "create_tensor: host allocation failed"); return nullptr; }
    size_t n = 1;
    for (int i = 0; i < ndim; i++) { impl->pub.shape[i] = shape[i]; n *= (size_t)(shape[i] > 0 ? shape[i] : 0); }
    impl->pub.ndim = ndim;
    impl->pub.size = n;
    impl->pub.dtype = dtype;
    impl->pub.data = nullptr;
    impl->magic = kTensorMagic;
    impl->refs.store(1);
    impl->base = nullptr;
    impl->device = current_device_index();
    impl->kind = kPool;
    return impl;
}

static void destroy_header(TensorImpl* impl) {
    impl->magic = 0;
    free(impl->pub.shape);
    delete impl;
}

static Tensor* allocate(const int* shape, int ndim, DataType dtype, bool zero) {
    DeviceState* st = acquire_device();
    if (!st) return nullptr;
    TensorImpl* impl = new_header(shape, ndim, dtype);
    if (!impl) return nullptr;
    size_t bytes = impl->pub.size * (size_t)dtype_bytes((int)dtype);
    if (bytes == 0) bytes = 16;                      // keep a valid, distinct pointer for empty tensors
    cudaStream_t s = current_stream();
    cudaError_t e;
    if (managed_mode()) {
        impl->kind = kManaged;
        e = cudaMallocManaged(&impl->pub.data, bytes);
        if (e == cudaSuccess && zero) e = cudaMemsetAsync(impl->pub.data, 0, bytes, s);     // on the stream that is synchronised next:
        if (e == cudaSuccess) e = cudaStreamSynchronize(s);                                 // the host may write into it right away
    } else {
        e = cudaMallocAsync(&impl->pub.data, bytes, s);
        if (e == cudaSuccess && zero) e = cudaMemsetAsync(impl->pub.data, 0, bytes, s);
    }
    if (!check_cuda(e, "create_tensor")) { destroy_header(impl); return nullptr; }
    return &impl->pub;
}

static void release(TensorImpl* impl) {
    while (impl) {
        if (impl->refs.fetch_sub(1) != 1) return;
        TensorImpl* base = impl->base;
        if (impl->kind == kPool || impl->kind == kManaged) {
            int restore = -1;
            cudaGetDevice(&restore);
            if (restore != impl->device) cudaSetDevice(impl->device);
            if (impl->kind == kPool) {
                const int dev = impl->device;
                cudaStream_t s = (dev >= 0 && dev < kMaxDevices)
                    ? (g_user_stream_set[dev] ? g_user_stream[dev] : g_devices[dev].own_stream) : nullptr;
                check_cuda(cudaFreeAsync(impl->pub.data, s), "free_tensor");
            } else {
                check_cuda(cudaFree(impl->pub.data), "free_tensor");
            }
            if (restore >= 0 && restore != impl->device) cudaSetDevice(restore);
        }
        destroy_header(impl);
        impl = base;                                  // a view drops its reference on the base
    }
}

void zero_fill(Tensor* t) {
    if (!t || !t->data || t->size == 0) return;
    if (!acquire_device()) return;
    cudaMemsetAsync(t->data, 0, t->size * (size_t)dtype_bytes((int)t->dtype), current_stream());
}

// ---- cosine table (tensor_ops.c:17-31, 763-807) ---------------------------------------------------
// Built on the host in double without fused multiply-adds (this translation unit's host code is
// compiled with -ffp-contract=off), uploaded once per device.
static double     g_cos_table[4097];
static std::once_flag g_cos_once;

static void build_cos_table() {
    const double pi = 3.141592653589793238462643383279502884197;
    const double two_pi = 2.0 * pi, half_pi = pi / 2.0;
    for (int i = 0; i <= 4096; i++) {
        double a = (double)i * two_pi / 4096;
        double sgn = 1.0;
        if (a > pi) a = two_pi - a;
        if (a > half_pi) { a = pi - a; sgn = -1.0; }
        double r;
        if (a < 0.785398163397448) {
            const double q = a * a;
            r = 1.0 + q * (-0.5 + q * (0.04166666666666666 + q * (-0.001388888888888889 + q * 0.000024801587301587302)));
        } else {
            const double t = half_pi - a, q = t * t;
            r = t * (1.0 + q * (-0.16666666666666666 + q * (0.008333333333333333 +
                q * (-0.0001984126984126984 + q * 0.0000027557319223985893))));
        }
        g_cos_table[i] = sgn * r;
    }
}

const double* cos_lut_device() {
    DeviceState* st = acquire_device();
    if (!st) return nullptr;
    if (st->cos_lut) return st->cos_lut;
    std::call_once(g_cos_once, build_cos_table);
    std::lock_guard<std::mutex> lock(g_device_mutex);
    if (st->cos_lut) return st->cos_lut;
    double* dev = nullptr;
    if (!TOPS_CUDA_OK(cudaMalloc(&dev, sizeof(g_cos_table)))) return nullptr;
    if (!TOPS_CUDA_OK(cudaMemcpy(dev, g_cos_table, sizeof(g_cos_table), cudaMemcpyHostToDevice))) { cudaFree(dev); return nullptr; }
    st->cos_lut = dev;
    return dev;
}

// ---- broadcast planning ---------------------------------------------------------------------------
bool plan_broadcast(const ShapeView& out, const ShapeView* ins, int n_in, Geometry* geom, Operand* ops) {
    constexpr int kMaxRank = 16;                     // the reference's MAX_NDIM (tensor_ops.c:10)
    const int ond = out.ndim > 0 ? out.ndim : 1;
    if (ond > kMaxRank) return false;
    long long osize[kMaxRank];
    for (int d = 0; d < ond; d++) osize[d] = out.ndim > 0 ? out.shape[d] : 1;

    long long stride[4][kMaxRank];
    if (n_in > 4) return false;
    bool any_bcast = false;
    for (int k = 0; k < n_in; k++) {
        ops[k].flat = (ins[k].size == out.size) ? 1 : 0;
        ops[k].nd = 0;
        // contiguous strides of the output: what a flat operand follows
        long long run = 1;
        for (int d = ond - 1; d >= 0; d--) { stride[k][d] = run; run *= osize[d]; }
        if (ops[k].flat) continue;
        any_bcast = true;
        const int ind = ins[k].ndim;
        // leading dims beyond the output rank must be 1
        for (int d = 0; d < ind - ond; d++) if (ins[k].shape[d] != 1) return false;
        run = 1;
        for (int d = ond - 1; d >= 0; d--) {
            const int id = d - (ond - ind);
            const long long sz = (id >= 0 && id < ind) ? ins[k].shape[id] : 1;
            if (sz == osize[d]) { stride[k][d] = run; run *= sz; }
            else if (sz == 1)   { stride[k][d] = 0; }
            else return false;
        }
    }

    if (!any_bcast) {
        geom->nd = 1;
        geom->size[0] = (uint32_t)(out.size < 0x7FFFFFFFull ? out.size : 0x7FFFFFFFull);
        geom->div[0].set(geom->size[0] ? geom->size[0] : 1);
        return true;
    }

    // Collapse: drop size-1 dims, merge neighbours that every operand walks contiguously.
    long long csize[kMaxRank];
    long long cstride[4][kMaxRank];
    int cnd = 0;
    for (int d = 0; d < ond; d++) {
        if (osize[d] == 1) continue;
        bool merge = cnd > 0;
        if (merge) for (int k = 0; k < n_in; k++) if (cstride[k][cnd - 1] != stride[k][d] * osize[d]) { merge = false; break; }
        if (merge) {
            csize[cnd - 1] *= osize[d];
            for (int k = 0; k < n_in; k++) cstride[k][cnd - 1] = stride[k][d];
        } else {
            csize[cnd] = osize[d];
            for (int k = 0; k < n_in; k++) cstride[k][cnd] = stride[k][d];
            cnd++;
        }
    }
    if (cnd == 0) { csize[0] = 1; for (int k = 0; k < n_in; k++) cstride[k][0] = 0; cnd = 1; }
    if (cnd > kMaxCollapsedDims) return false;
    geom->nd = cnd;
    for (int d = 0; d < cnd; d++) {
        if (csize[d] > 0x7FFFFFFFll) return false;
        geom->size[d] = (uint32_t)csize[d];
        geom->div[d].set((uint32_t)csize[d]);
    }
    for (int k = 0; k < n_in; k++) {
        ops[k].nd = cnd;
        for (int d = 0; d < cnd; d++) {
            if (cstride[k][d] > 0x7FFFFFFFll) return false;
            ops[k].stride[d] = (int)cstride[k][d];
        }
    }
    return true;
}

}  // namespace tops

using namespace tops;

// ---- exported: reference entry points -----------------------------------------------------------------
TOPS_API Tensor* create_tensor(int* shape, int ndim, DataType dtype) { return allocate(shape, ndim, dtype, true); }

TOPS_API void free_tensor(Tensor* tensor) {
    if (!tensor) return;
    TensorImpl* impl = impl_of(tensor);
    if (!impl) { set_error(TOPS_ERR_INVALID, "free_tensor: not a tensor created by this library"); return; }
    release(impl);
}

TOPS_API void init_cos_lut(void) { (void)cos_lut_device(); }

TOPS_API void flatten_forward(const Tensor* input, Tensor* output) {
    if (!input || !output || !input->data || !output->data || input->size != output->size) {
        set_error(TOPS_ERR_INVALID, "flatten_forward: null tensor or size mismatch");
        zero_fill(output);
        return;
    }
    if (!acquire_device()) return;
    const size_t bytes = input->size * (size_t)dtype_bytes((int)input->dtype);
    if (bytes && input->data != output->data)
        TOPS_CUDA_OK(cudaMemcpyAsync(output->data, input->data, bytes, cudaMemcpyDeviceToDevice, current_stream()));
    finish_op();
}

TOPS_API void reshape_forward(const Tensor* input, Tensor* output) { flatten_forward(input, output); }

// ---- exported: additive interface -------------------------------------------------------------------------
TOPS_API int tops_last_error(void) { return g_error.load(); }
TOPS_API const char* tops_last_error_message(void) { return g_error_message; }
TOPS_API void tops_clear_error(void) {
    std::lock_guard<std::mutex> lock(g_error_mutex);
    g_error.store(TOPS_OK);
    g_error_message[0] = 0;
}

TOPS_API int tops_device_count(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) { cudaGetLastError(); return 0; }
    return n;
}
TOPS_API int tops_set_device(int device) {
    if (device < 0 || device >= kMaxDevices || device >= tops_device_count()) {
        set_error(TOPS_ERR_NO_DEVICE, "tops_set_device: device %d not available", device);
        return TOPS_ERR_NO_DEVICE;
    }
    t_device = device;
    return acquire_device() ? TOPS_OK : tops_last_error();
}
TOPS_API int tops_get_device(void) { return current_device_index(); }
TOPS_API void* tops_get_stream(void) { return acquire_device() ? (void*)current_stream() : nullptr; }
TOPS_API int tops_set_stream(void* cuda_stream) {
    if (!acquire_device()) return tops_last_error();
    const int dev = current_device_index();
    g_user_stream[dev] = (cudaStream_t)cuda_stream;
    g_user_stream_set[dev] = cuda_stream != nullptr;
    return TOPS_OK;
}
TOPS_API int tops_sync(void) {
    if (!acquire_device()) return tops_last_error();
    const bool ok = TOPS_CUDA_OK(cudaStreamSynchronize(current_stream()));
    poll_device_status();
    return ok ? tops_last_error() : tops_last_error();
}
TOPS_API int tops_set_memory_mode(int managed) { g_managed.store(managed ? 1 : 0); return TOPS_OK; }

// ---- stream capture: a fixed sequence of operator calls as one CUDA graph ---------------------------------------
// Everything an operator enqueues (kernels, memsets, its stream-ordered scratch allocations and their releases)
// lands on the current stream, so capturing that stream while the calls are repeated records the whole sequence;
// launching the instantiated graph then costs one driver call instead of one per kernel.
struct CapturedGraph { cudaGraphExec_t exec; int device; };

TOPS_API int tops_capture_begin(void) {
    if (!acquire_device()) return tops_last_error();
    if (managed_mode()) { set_error(TOPS_ERR_UNSUPPORTED, "tops_capture_begin: managed-memory mode synchronises after every operator"); return tops_last_error(); }
    return TOPS_CUDA_OK(cudaStreamBeginCapture(current_stream(), cudaStreamCaptureModeRelaxed)) ? TOPS_OK : tops_last_error();
}

TOPS_API void* tops_capture_end(void) {
    if (!acquire_device()) return nullptr;
    cudaGraph_t graph = nullptr;
    const cudaError_t e = cudaStreamEndCapture(current_stream(), &graph);
    if (e != cudaSuccess || !graph) {
        cudaGetLastError();
        set_error(TOPS_ERR_CUDA, "tops_capture_end: the sequence could not be captured (%s)", cudaGetErrorString(e));
        return nullptr;
    }
    cudaGraphExec_t exec = nullptr;
    const bool ok = TOPS_CUDA_OK(cudaGraphInstantiate(&exec, graph, 0));
    cudaGraphDestroy(graph);
    if (!ok) return nullptr;
    CapturedGraph* out = new (std::nothrow) CapturedGraph{exec, current_device_index()};
    if (!out) { cudaGraphExecDestroy(exec); set_error(TOPS_ERR_OOM, "tops_capture_end: host allocation failed"); }
    return out;
}

TOPS_API int tops_capture_launch(void* captured) {
    CapturedGraph* g = (CapturedGraph*)captured;
    if (!g) { set_error(TOPS_ERR_INVALID, "tops_capture_launch: null graph"); return tops_last_error(); }
    if (!acquire_device()) return tops_last_error();
    if (g->device != current_device_index()) { set_error(TOPS_ERR_INVALID, "tops_capture_launch: captured on device %d", g->device); return tops_last_error(); }
    return TOPS_CUDA_OK(cudaGraphLaunch(g->exec, current_stream())) ? TOPS_OK : tops_last_error();
}

TOPS_API void tops_capture_free(void* captured) {
    CapturedGraph* g = (CapturedGraph*)captured;
    if (!g) return;
    cudaGraphExecDestroy(g->exec);
    delete g;
}

TOPS_API Tensor* tops_create_uninit(const int* shape, int ndim, DataType dtype) { return allocate(shape, ndim, dtype, false); }

TOPS_API Tensor* tops_wrap(void* device_ptr, const int* shape, int ndim, DataType dtype) {
    TensorImpl* impl = new_header(shape, ndim, dtype);
    if (!impl) return nullptr;
    impl->kind = kWrapped;
    impl->pub.data = device_ptr;
    return &impl->pub;
}

TOPS_API Tensor* tops_view(Tensor* base, const int* shape, int ndim) {
    TensorImpl* b = impl_of(base);
    if (!b) { set_error(TOPS_ERR_INVALID, "tops_view: not a tensor created by this library"); return nullptr; }
    TensorImpl* impl = new_header(shape, ndim, base->dtype);
    if (!impl) return nullptr;
    if (impl->pub.size != base->size) {
        destroy_header(impl);
        set_error(TOPS_ERR_INVALID, "tops_view: element count differs from the base tensor");
        return nullptr;
    }
    impl->kind = kView;
    impl->pub.data = base->data;
    impl->device = b->device;
    impl->base = b;
    b->refs.fetch_add(1);
    return &impl->pub;
}

TOPS_API Tensor* tops_slice_rows(Tensor* base, int row_begin, int row_count) {
    TensorImpl* b = impl_of(base);
    if (!b || base->ndim < 1 || row_begin < 0 || row_count < 0 || row_begin + row_count > base->shape[0]) {
        set_error(TOPS_ERR_INVALID, "tops_slice_rows: bad tensor or row range");
        return nullptr;
    }
    int shape[16];
    if (base->ndim > 16) { set_error(TOPS_ERR_INVALID, "tops_slice_rows: rank above 16"); return nullptr; }
    for (int d = 0; d < base->ndim; d++) shape[d] = base->shape[d];
    shape[0] = row_count;
    TensorImpl* impl = new_header(shape, base->ndim, base->dtype);
    if (!impl) return nullptr;
    const size_t row_elems = base->shape[0] ? base->size / (size_t)base->shape[0] : 0;
    impl->kind = kView;
    impl->pub.data = (char*)base->data + (size_t)row_begin * row_elems * (size_t)dtype_bytes((int)base->dtype);
    impl->device = b->device;
    impl->base = b;
    b->refs.fetch_add(1);
    return &impl->pub;
}

TOPS_API void tops_retain(Tensor* tensor) {
    if (TensorImpl* impl = impl_of(tensor)) impl->refs.fetch_add(1);
}

TOPS_API size_t tops_dtype_size(DataType dtype) { return (size_t)dtype_bytes((int)dtype); }

static bool transfer_args_ok(const Tensor* t, const void* host, size_t nbytes, const char* who) {
    if (!t || !t->data || (!host && nbytes)) { set_error(TOPS_ERR_INVALID, "%s: null argument", who); return false; }
    if (nbytes > t->size * (size_t)dtype_bytes((int)t->dtype)) {
        set_error(TOPS_ERR_INVALID, "%s: %zu bytes exceed the tensor", who, nbytes);
        return false;
    }
    return true;
}

TOPS_API int tops_upload(Tensor* dst, const void* host, size_t nbytes) {
    if (!transfer_args_ok(dst, host, nbytes, "tops_upload") || !acquire_device()) return tops_last_error();
    if (nbytes == 0) return TOPS_OK;
    return TOPS_CUDA_OK(cudaMemcpyAsync(dst->data, host, nbytes, cudaMemcpyHostToDevice, current_stream())) ? TOPS_OK : tops_last_error();
}
TOPS_API int tops_download_async(const Tensor* src, void* host, size_t nbytes) {
    if (!transfer_args_ok(src, host, nbytes, "tops_download") || !acquire_device()) return tops_last_error();
    if (nbytes == 0) return TOPS_OK;
    return TOPS_CUDA_OK(cudaMemcpyAsync(host, src->data, nbytes, cudaMemcpyDeviceToHost, current_stream())) ? TOPS_OK : tops_last_error();
}
TOPS_API int tops_download(const Tensor* src, void* host, size_t nbytes) {
    const int rc = tops_download_async(src, host, nbytes);
    if (rc != TOPS_OK) return rc;
    const bool ok = TOPS_CUDA_OK(cudaStreamSynchronize(current_stream()));
    poll_device_status();
    return ok ? tops_last_error() : tops_last_error();
}
TOPS_API void* tops_host_alloc(size_t nbytes) {
    if (!acquire_device()) return nullptr;
    void* p = nullptr;
    if (!TOPS_CUDA_OK(cudaHostAlloc(&p, nbytes ? nbytes : 1, cudaHostAllocDefault))) return nullptr;
    return p;
}
TOPS_API void tops_host_free(void* host) { if (host) cudaFreeHost(host); }

TOPS_API const char* tops_version(void) { return "tensor_ops_b200 0.1 (sm_100a)"; }

// Host-only view of the broadcast planner (no CUDA call), so its index logic can be tested on a
// machine without a GPU.  Fills nd, sizes[nd], strides[nd] and flat for ONE operand.
TOPS_API int tops_debug_plan_broadcast(const int* out_shape, int out_ndim, const int* in_shape, int in_ndim,
                                       int* nd, unsigned* sizes, int* strides, int* flat) {
    size_t osz = 1, isz = 1;
    for (int i = 0; i < out_ndim; i++) osz *= (size_t)out_shape[i];
    for (int i = 0; i < in_ndim; i++) isz *= (size_t)in_shape[i];
    Geometry g;
    Operand op;
    const ShapeView out{out_shape, out_ndim, osz}, in{in_shape, in_ndim, isz};
    if (!plan_broadcast(out, &in, 1, &g, &op)) return 0;
    *nd = g.nd;
    *flat = op.flat;
    for (int d = 0; d < g.nd; d++) { sizes[d] = g.size[d]; strides[d] = op.flat ? 0 : op.stride[d]; }
    return 1;
}

// ---- device status word ------------------------------------------------------------------------------------
// One int in pinned, device-mapped host memory.  Kernels with bounded waits set it when a wait
// gives up; the host looks at it whenever it synchronises and turns it into TOPS_ERR_DEVICE_TIMEOUT.
namespace tops {
static int* g_status_host = nullptr;
static std::once_flag g_status_once;

int* device_status_word() {
    std::call_once(g_status_once, [] {
        if (cudaHostAlloc((void**)&g_status_host, sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) {
            g_status_host = nullptr;
            cudaGetLastError();
            return;
        }
        *g_status_host = 0;
    });
    if (!g_status_host) return nullptr;
    int* dev = nullptr;
    if (cudaHostGetDevicePointer((void**)&dev, g_status_host, 0) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return dev;
}

// The same pointer, but only if an earlier call already created the word: never allocates.
int* device_status_word_if_created() {
    if (!g_status_host) return nullptr;
    int* dev = nullptr;
    if (cudaHostGetDevicePointer((void**)&dev, g_status_host, 0) != cudaSuccess) { cudaGetLastError(); return nullptr; }
    return dev;
}

void poll_device_status() {
    if (g_status_host && *(volatile int*)g_status_host) {
        *(volatile int*)g_status_host = 0;
        set_error(TOPS_ERR_DEVICE_TIMEOUT, "a bounded device-side wait expired inside a tensor-core kernel");
    }
}
}  // namespace tops
