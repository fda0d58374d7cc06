// Elementwise engine: every unary / binary / Q / DQ kernel is one instantiation of ew_kernel
// around a small "body" functor.  A thread owns runs of V consecutive output elements (V chosen
// so the widest stream moves 16 bytes per access), walks them grid-stride, and fetches each
// operand either as one vector (flat operands, or broadcast operands whose run stays inside the
// innermost collapsed dimension) or element by element at run boundaries.
#pragma once

#include "common.cuh"

namespace tops {

constexpr int kEwThreads = 256;

// ---- raw vector moves ---------------------------------------------------------------------------------
template <int BYTES> __device__ __forceinline__ void load_bytes(const void* src, void* dst) {
    if constexpr (BYTES == 1)       *(uint8_t*)dst  = *(const uint8_t*)src;
    else if constexpr (BYTES == 2)  *(uint16_t*)dst = *(const uint16_t*)src;
    else if constexpr (BYTES == 4)  *(uint32_t*)dst = *(const uint32_t*)src;
    else if constexpr (BYTES == 8)  *(uint2*)dst    = *(const uint2*)src;
    else {
        static_assert(BYTES % 16 == 0, "vector width");
        #pragma unroll
        for (int k = 0; k < BYTES / 16; k++) ((uint4*)dst)[k] = ((const uint4*)src)[k];
    }
}
// Streaming variants for data touched exactly once (evict-first in L2, no L1 allocation).
template <int BYTES> __device__ __forceinline__ void load_bytes_stream(const void* src, void* dst) {
    if constexpr (BYTES == 4)       *(uint32_t*)dst = __ldcs((const uint32_t*)src);
    else if constexpr (BYTES == 8)  *(uint2*)dst    = __ldcs((const uint2*)src);
    else if constexpr (BYTES >= 16) {
        #pragma unroll
        for (int k = 0; k < BYTES / 16; k++) ((uint4*)dst)[k] = __ldcs(((const uint4*)src) + k);
    } else load_bytes<BYTES>(src, dst);
}
template <int BYTES> __device__ __forceinline__ void store_bytes_stream(void* dst, const void* src) {
    if constexpr (BYTES == 1)       *(uint8_t*)dst  = *(const uint8_t*)src;
    else if constexpr (BYTES == 2)  *(uint16_t*)dst = *(const uint16_t*)src;
    else if constexpr (BYTES == 4)  __stcs((uint32_t*)dst, *(const uint32_t*)src);
    else if constexpr (BYTES == 8)  __stcs((uint2*)dst, *(const uint2*)src);
    else {
        #pragma unroll
        for (int k = 0; k < BYTES / 16; k++) __stcs(((uint4*)dst) + k, ((const uint4*)src)[k]);
    }
}

template <typename S, int V> struct alignas(sizeof(S) * V >= 16 ? 16 : sizeof(S) * V) Run { S v[V]; };

// Fetch V elements of an operand for output indices [i0, i0 + nv).
// `vec_ok`: the operand's base pointer is aligned to V elements.
template <int DT, int V>
__device__ __forceinline__ void fetch(const Geometry& g, const Operand& op, uint32_t i0, uint32_t nv, bool vec_ok,
                                      Run<typename Storage<DT>::type, V>& out) {
    using S = typename Storage<DT>::type;
    const S* base = (const S*)op.ptr;
    if (op.flat) {
        if (nv == V && vec_ok) { load_bytes_stream<sizeof(S) * V>(base + i0, &out); return; }
        #pragma unroll
        for (int j = 0; j < V; j++) out.v[j] = (uint32_t)j < nv ? base[i0 + j] : S(0);
        return;
    }
    uint32_t pos;
    const uint32_t off = operand_offset(g, op, i0, pos);
    const int inner = op.stride[g.nd - 1];
    if (pos + V <= g.size[g.nd - 1]) {               // the whole run sits in the innermost dimension
        if (inner == 0) {
            const S s = base[off];
            #pragma unroll
            for (int j = 0; j < V; j++) out.v[j] = s;
        } else if (vec_ok && (off % V) == 0) {
            load_bytes<sizeof(S) * V>(base + off, &out);
        } else {
            #pragma unroll
            for (int j = 0; j < V; j++) out.v[j] = base[off + j];
        }
        return;
    }
    #pragma unroll
    for (int j = 0; j < V; j++) {
        uint32_t p;
        out.v[j] = (uint32_t)j < nv ? base[operand_offset(g, op, i0 + j, p)] : S(0);
    }
}

template <int DT, int V>
__device__ __forceinline__ void put(void* out_ptr, uint32_t i0, uint32_t nv, bool vec_ok,
                                    const Run<typename Storage<DT>::type, V>& r) {
    using S = typename Storage<DT>::type;
    S* base = (S*)out_ptr;
    if (nv == V && vec_ok) { store_bytes_stream<sizeof(S) * V>(base + i0, &r); return; }
    #pragma unroll
    for (int j = 0; j < V; j++) if ((uint32_t)j < nv) base[i0 + j] = r.v[j];
}

// ---- the kernel ----------------------------------------------------------------------------------------
template <class Body>
__global__ void __launch_bounds__(kEwThreads) ew_kernel(const Body body, const uint32_t n) {
    constexpr uint32_t V = Body::kV;
    const uint32_t runs = (n + V - 1) / V;
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += step) {
        const uint32_t i0 = r * V;
        const uint32_t left = n - i0;
        body(i0, left < V ? left : V);
    }
}

constexpr int vec_width(int bytes_a, int bytes_b, int bytes_c) {
    int m = bytes_a > bytes_b ? bytes_a : bytes_b;
    m = m > bytes_c ? m : bytes_c;
    return 16 / m;
}

inline bool aligned_to(const void* p, size_t bytes) { return ((uintptr_t)p % bytes) == 0; }

// Launches `make_body(geometry, operands, out_ptr)` over the output, in slabs of < 2^31 elements.
// Slabs cut the outermost collapsed dimension, so operand offsets advance by stride[0].
template <class MakeBody>
bool launch_elementwise(const char* name, const Geometry& geom, Operand* ops, const int* op_bytes, int n_ops,
                        void* out, int out_bytes, size_t total, MakeBody&& make_body) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    if (total == 0) return true;
    cudaStream_t stream = current_stream();
    bool all_flat = true;
    for (int k = 0; k < n_ops; k++) all_flat = all_flat && ops[k].flat;

    const size_t kSlabMax = 0x7FFFFF00ull;               // multiple of 256: slabs keep vector alignment
    size_t inner = 1;                                    // elements per index of the outermost dim
    if (!all_flat) for (int d = 1; d < geom.nd; d++) inner *= geom.size[d];
    if (inner > kSlabMax) { set_error(TOPS_ERR_UNSUPPORTED, "%s: broadcast row of %zu elements is too long", name, inner); return false; }
    const size_t rows_total = all_flat ? total : geom.size[0];
    const size_t rows_per_slab = all_flat ? kSlabMax : (kSlabMax / inner ? kSlabMax / inner : 1);

    for (size_t row = 0; row < rows_total; row += rows_per_slab) {
        const size_t rows = (rows_total - row < rows_per_slab) ? rows_total - row : rows_per_slab;
        const size_t n = all_flat ? rows : rows * inner;
        const size_t first = all_flat ? row : row * inner;
        Geometry g = geom;
        if (all_flat) { g.nd = 1; g.size[0] = (uint32_t)n; g.div[0].set((uint32_t)n); }
        else          { g.size[0] = (uint32_t)rows; g.div[0].set((uint32_t)rows); }
        Operand local[4];
        for (int k = 0; k < n_ops; k++) {
            local[k] = ops[k];
            const size_t off = ops[k].flat ? first : row * (size_t)ops[k].stride[0];
            local[k].ptr = (const char*)ops[k].ptr + off * (size_t)op_bytes[k];
        }
        void* out_slab = (char*)out + first * (size_t)out_bytes;
        auto body = make_body(g, local, out_slab);
        using Body = decltype(body);
        const size_t runs = (n + Body::kV - 1) / Body::kV;
        const int grid = grid_for(runs, kEwThreads, st->sm_count, 8);
        ew_kernel<Body><<<grid, kEwThreads, 0, stream>>>(body, (uint32_t)n);
        if (!TOPS_CHECK_LAUNCH(name)) return false;
    }
    return true;
}

}  // namespace tops
