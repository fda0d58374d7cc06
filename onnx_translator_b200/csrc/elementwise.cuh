// Elementwise engine: every unary / binary / Q / DQ kernel is one instantiation of ew_kernel
// around a small "body" functor.  A thread owns runs of V consecutive output elements (V chosen
// so the widest stream moves 16 bytes per access) and walks them grid-stride.
//
// Typed bodies see the output through a fixed three-level geometry [c0][c1][c2] (collapsed
// dimensions, outermost first, padded in front).  An operand is three element strides: a dense
// operand has (s1*s2, s2, 1) so its offset IS the output index, a broadcast operand has zeros.
// Coordinates are computed once per run with two multiply-high divisions and shared by all
// operands.  Shapes that do not collapse to three dimensions, and dtype combinations without a
// typed body, take the generic bodies (any rank up to 16, one element per run).
#pragma once

#include "common.cuh"

namespace tops {

constexpr int kEwThreads = 256;
constexpr int kEwCtasPerSm = 8;

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
// Streaming variants for data touched exactly once (evict-first).
template <int BYTES> __device__ __forceinline__ void load_bytes_stream(const void* src, void* dst) {
    if constexpr (BYTES == 4)       *(uint32_t*)dst = __ldcs((const uint32_t*)src);
    else if constexpr (BYTES == 8)  *(uint2*)dst    = __ldcs((const uint2*)src);
    else if constexpr (BYTES >= 16) {
        static_assert(BYTES % 16 == 0, "vector width");
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
        static_assert(BYTES % 16 == 0, "vector width");
        #pragma unroll
        for (int k = 0; k < BYTES / 16; k++) __stcs(((uint4*)dst) + k, ((const uint4*)src)[k]);
    }
}

template <typename S, int V> struct alignas(sizeof(S) * V >= 16 ? 16 : sizeof(S) * V) Run { S v[V]; };

// ---- three-level geometry ---------------------------------------------------------------------------------
struct Geo3 {
    uint32_t s1 = 0x80000000u, s2 = 0x80000000u;   // sizes of the two inner levels (padding: 2^31)
    FastDiv d1, d2;
    int simple = 1;                                // every operand dense: offsets equal the index
};
struct Op3 {
    const void* ptr = nullptr;
    uint32_t st0 = 0, st1 = 0, st2 = 1;
};
struct Coord3 { uint32_t c0, c1, c2; };

__device__ __forceinline__ Coord3 coords_of(const Geo3& g, uint32_t i) {
    Coord3 c;
    const uint32_t t = g.d2.div(i);
    c.c2 = i - t * g.s2;
    c.c0 = g.d1.div(t);
    c.c1 = t - c.c0 * g.s1;
    return c;
}
__device__ __forceinline__ uint32_t offset_of(const Op3& op, const Coord3& c) {
    return c.c0 * op.st0 + c.c1 * op.st1 + c.c2 * op.st2;
}

// Fetch a whole run.  ALIGNED: the run lies inside one innermost row and vector accesses are
// aligned (checked on the host).  Otherwise each element is addressed on its own.
template <int DT, int V, bool ALIGNED>
__device__ __forceinline__ void fetch3(const Geo3& g, const Op3& op, uint32_t i0, uint32_t nv, const Coord3& c,
                                       Run<typename Storage<DT>::type, V>& out) {
    using S = typename Storage<DT>::type;
    const S* base = (const S*)op.ptr;
    if (ALIGNED && nv == V) {
        if (g.simple) { load_bytes_stream<sizeof(S) * V>(base + i0, &out); return; }
        const uint32_t off = offset_of(op, c);
        if (op.st2 == 0) {
            const S s = base[off];
            #pragma unroll
            for (int j = 0; j < V; j++) out.v[j] = s;
        } else if (op.st0 | op.st1) {
            load_bytes_stream<sizeof(S) * V>(base + off, &out);      // a big operand: touched once
        } else {
            load_bytes<sizeof(S) * V>(base + off, &out);             // a small vector: keep it cached
        }
        return;
    }
    #pragma unroll
    for (int j = 0; j < V; j++) {
        S s = S(0);
        if ((uint32_t)j < nv) s = g.simple ? base[i0 + j] : base[offset_of(op, coords_of(g, i0 + j))];
        out.v[j] = s;
    }
}

template <int DT, int V, bool ALIGNED>
__device__ __forceinline__ void put3(void* out_ptr, uint32_t i0, uint32_t nv, const Run<typename Storage<DT>::type, V>& r) {
    using S = typename Storage<DT>::type;
    S* base = (S*)out_ptr;
    if (ALIGNED && nv == V) { store_bytes_stream<sizeof(S) * V>(base + i0, &r); return; }
    #pragma unroll
    for (int j = 0; j < V; j++) if ((uint32_t)j < nv) base[i0 + j] = r.v[j];
}

// ---- packed decode / encode of whole runs --------------------------------------------------------------------
template <int DT, int V>
__device__ __forceinline__ void decode_floats(const Run<typename Storage<DT>::type, V>& r, float (&f)[V]) {
    if constexpr (DT == DTYPE_FLOAT16 && V % 2 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 2) {
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&r.v[j]));
            f[j] = p.x; f[j + 1] = p.y;
        }
    } else if constexpr (DT == DTYPE_FLOAT8_E4M3 && V % 2 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 2) {                    // two codes per hardware convert
            const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(*reinterpret_cast<const uint16_t*>(&r.v[j]), __NV_E4M3);
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&h));
            f[j] = p.x; f[j + 1] = p.y;
        }
    } else if constexpr (DT == DTYPE_FLOAT8_E5M2 && V % 2 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 2) {                    // an e5m2 code is the upper byte of a float16
            const uint32_t h = __byte_perm((uint32_t)*reinterpret_cast<const uint16_t*>(&r.v[j]), 0u, 0x1404);
            const float2 p = __half22float2(*reinterpret_cast<const __half2*>(&h));
            f[j] = p.x; f[j + 1] = p.y;
        }
    } else if constexpr ((DT == DTYPE_INT8 || DT == DTYPE_UINT8) && V % 4 == 0) {
        // 8-bit integers to float without the conversion unit: the byte becomes the low mantissa
        // byte of 2^23 (signed bytes are first biased by 128), then the constant is subtracted
        #pragma unroll
        for (int j = 0; j < V; j += 4) {
            uint32_t w = *reinterpret_cast<const uint32_t*>(&r.v[j]);
            if (DT == DTYPE_INT8) w ^= 0x80808080u;
            const float bias = DT == DTYPE_INT8 ? 8388736.0f : 8388608.0f;
            f[j]     = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7540)), bias);
            f[j + 1] = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7541)), bias);
            f[j + 2] = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7542)), bias);
            f[j + 3] = __fsub_rn(__uint_as_float(__byte_perm(w, 0x4B000000u, 0x7543)), bias);
        }
    } else {
        #pragma unroll
        for (int j = 0; j < V; j++) f[j] = to_f32<DT>(r.v[j]);
    }
}

// Pairs of float32 -> packed 16-bit codes: one hardware convert for both lanes, then the
// reference's deviations (NaN codes, fp16 flush below 2^-24) on the rare lanes that need them.
__device__ __forceinline__ uint32_t encode_f16x2(float lo, float hi) {
    const uint32_t bl = f32_bits(lo), bh = f32_bits(hi);
    const uint32_t ml = bl & 0x7FFFFFFFu, mh = bh & 0x7FFFFFFFu;
    // magnitudes below 2^-24 become a signed zero first (the hardware would round [2^-25, 2^-24) up)
    const float fl = ml < 0x33800000u ? __uint_as_float(bl & 0x80000000u) : lo;
    const float fh = mh < 0x33800000u ? __uint_as_float(bh & 0x80000000u) : hi;
    const __half2 h = __floats2half2_rn(fl, fh);
    uint32_t packed = *reinterpret_cast<const uint32_t*>(&h);
    if ((ml > 0x7F800000u) | (mh > 0x7F800000u))               // NaN keeps its sign and gets payload 0x3FF
        packed = (uint32_t)encode_f16(lo) | ((uint32_t)encode_f16(hi) << 16);
    return packed;
}
__device__ __forceinline__ uint32_t encode_bf16x2(float lo, float hi) {
    const __nv_bfloat162 b = __floats2bfloat162_rn(lo, hi);
    uint32_t packed = *reinterpret_cast<const uint32_t*>(&b);
    if ((lo != lo) | (hi != hi)) packed = (uint32_t)encode_bf16(lo) | ((uint32_t)encode_bf16(hi) << 16);
    return packed;
}

template <int DT, int V>
__device__ __forceinline__ void encode_floats(const float (&f)[V], Run<typename Storage<DT>::type, V>& r) {
    if constexpr (DT == DTYPE_FLOAT16 && V % 2 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 2) *reinterpret_cast<uint32_t*>(&r.v[j]) = encode_f16x2(f[j], f[j + 1]);
    } else if constexpr (DT == DTYPE_BFLOAT16 && V % 2 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 2) *reinterpret_cast<uint32_t*>(&r.v[j]) = encode_bf16x2(f[j], f[j + 1]);
    } else {
        #pragma unroll
        for (int j = 0; j < V; j++) r.v[j] = from_f32<DT>(f[j]);
    }
}

// Four int32 -> four saturated 8-bit codes in one word (two cvt.pack instructions).
__device__ __forceinline__ uint32_t pack_sat_s8x4(int a0, int a1, int a2, int a3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(a3), "r"(a2), "r"(0));
    asm("cvt.pack.sat.s8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(a1), "r"(a0), "r"(hi));
    return out;
}
__device__ __forceinline__ uint32_t pack_sat_u8x4(int a0, int a1, int a2, int a3) {
    uint32_t hi, out;
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(hi) : "r"(a3), "r"(a2), "r"(0));
    asm("cvt.pack.sat.u8.s32.b32 %0, %1, %2, %3;" : "=r"(out) : "r"(a1), "r"(a0), "r"(hi));
    return out;
}

template <int DT, int V>
__device__ __forceinline__ void encode_ints(const int (&v)[V], Run<typename Storage<DT>::type, V>& r) {
    if constexpr (DT == DTYPE_INT8 && V % 4 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 4) *reinterpret_cast<uint32_t*>(&r.v[j]) = pack_sat_s8x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else if constexpr (DT == DTYPE_UINT8 && V % 4 == 0) {
        #pragma unroll
        for (int j = 0; j < V; j += 4) *reinterpret_cast<uint32_t*>(&r.v[j]) = pack_sat_u8x4(v[j], v[j + 1], v[j + 2], v[j + 3]);
    } else {
        #pragma unroll
        for (int j = 0; j < V; j++) r.v[j] = from_i32<DT>(v[j]);
    }
}

// ---- the kernels ---------------------------------------------------------------------------------------
// Run kernel: a thread owns one run of V consecutive outputs per step (generic bodies, V = 1).
// Both kernels may be launched with programmatic stream serialisation: the grid is then scheduled
// while the previous kernel of the stream drains, and waits here -- before its first access to
// memory -- until that kernel has completed and its writes are visible.  Without the launch
// attribute the wait returns at once.
// Once past the wait a block lets the NEXT kernel of the stream be scheduled onto free SMs (it will
// sit in its own wait until this grid has finished).
__device__ __forceinline__ void wait_for_previous_kernel() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <class Body>
__global__ void __launch_bounds__(kEwThreads) ew_kernel(const Body body, const uint32_t n) {
    wait_for_previous_kernel();
    constexpr uint32_t V = Body::kV;
    const uint32_t runs = (n + V - 1) / V;
    const uint32_t step = gridDim.x * blockDim.x;
    for (uint32_t r = blockIdx.x * blockDim.x + threadIdx.x; r < runs; r += step) {
        const uint32_t i0 = r * V;
        const uint32_t left = n - i0;
        body(i0, left < V ? left : V);
    }
}

// Tile kernel (typed bodies): a warp owns tiles of 32 * V * G consecutive outputs.  Within a tile
// lane l takes the runs l, l + 32, ..., l + 32 (G - 1), so every access of the warp covers one
// contiguous span (512 bytes for the widest stream, whose runs are 16 bytes) whatever the other
// streams' widths, and the loads of all G runs are issued before the first result is needed.
template <class Body>
__global__ void __launch_bounds__(kEwThreads) ew_kernel_tiled(const Body body, const uint32_t n) {
    wait_for_previous_kernel();
    constexpr uint32_t V = Body::kV, G = Body::kGroups, TILE = 32u * V * G;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, warps = (gridDim.x * blockDim.x) >> 5;
    for (uint32_t base = warp * TILE; base < n; base += warps * TILE) {          // n < 2^31 and warps * TILE < 2^30
        typename Body::Regs regs[G];
        #pragma unroll
        for (uint32_t j = 0; j < G; j++) {
            const uint32_t i0 = base + (j * 32u + lane) * V;
            if (i0 < n) body.load(i0, n - i0 < V ? n - i0 : V, regs[j]);
        }
        #pragma unroll
        for (uint32_t j = 0; j < G; j++) {
            const uint32_t i0 = base + (j * 32u + lane) * V;
            if (i0 < n) body.finish(i0, n - i0 < V ? n - i0 : V, regs[j]);
        }
    }
}

// Elements per run: the narrowest stream would like 16 bytes per access; `cap_bytes` bounds what the
// widest stream then moves per run (16 = one vector access per lane for the widest stream).
//
// Which kernel and which widths a body uses is decided by measurement on B200 (A/B builds over the
// 95-launch sweep and the 8192 x 8192 quantize cases):
//   * same-width add / sub / mul, unary ops: run kernel, 16-byte runs (5.4-5.9 TB/s; the tile kernel
//     costs registers, hence occupancy, and is 10-15 % slower for the 16-bit types);
//   * operands of different widths (int8 + float32, int32 + float16 -> float64), dequantize: tile kernel
//     with two runs per lane (+10-17 %: every access of the warp is one contiguous span);
//   * float32 / float64 division: tile kernel with four runs per lane (+20 %: more divisions in flight);
//   * quantize to 8 bits: run kernel with 64-byte runs of float32 (16-byte stores of the codes).
constexpr int vec_width(int bytes_a, int bytes_b, int bytes_c, int cap_bytes = 16) {
    int lo = bytes_a < bytes_b ? bytes_a : bytes_b;
    lo = lo < bytes_c ? lo : bytes_c;
    int hi = bytes_a > bytes_b ? bytes_a : bytes_b;
    hi = hi > bytes_c ? hi : bytes_c;
    int v = 16 / lo;
    while (v > 1 && v * hi > cap_bytes) v /= 2;
    return v;
}

inline bool aligned_to(const void* p, size_t bytes) { return ((uintptr_t)p % bytes) == 0; }

// One slab (< 2^31 elements) of an elementwise launch.
struct Slab {
    Geometry geom;          // general geometry (generic bodies)
    Operand ops[4];
    Geo3 geo3;              // three-level geometry (typed bodies); valid when `fits3`
    Op3 ops3[4];
    bool fits3 = false;
    void* out = nullptr;
    size_t n = 0;
};

// Walks the output in slabs that cut the outermost collapsed dimension and calls `emit(slab)`.
template <class Emit>
bool for_each_slab(const char* name, const Geometry& geom, const Operand* ops, const int* op_bytes, int n_ops,
                   void* out, int out_bytes, size_t total, Emit&& emit) {
    if (total == 0) return true;
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
        Slab s;
        s.n = all_flat ? rows : rows * inner;
        const size_t first = all_flat ? row : row * inner;
        s.geom = geom;
        if (all_flat) { s.geom.nd = 1; s.geom.size[0] = (uint32_t)s.n; s.geom.div[0].set((uint32_t)s.n); }
        else          { s.geom.size[0] = (uint32_t)rows; s.geom.div[0].set((uint32_t)rows); }
        for (int k = 0; k < n_ops; k++) {
            s.ops[k] = ops[k];
            const size_t off = ops[k].flat ? first : row * (size_t)ops[k].stride[0];
            s.ops[k].ptr = (const char*)ops[k].ptr + off * (size_t)op_bytes[k];
        }
        s.out = (char*)out + first * (size_t)out_bytes;

        // three-level view: pad in front with 2^31-sized levels that no index reaches
        const int nd = s.geom.nd;
        s.fits3 = nd <= 3;
        if (s.fits3) {
            s.geo3.simple = all_flat ? 1 : 0;
            s.geo3.s2 = s.geom.size[nd - 1];
            s.geo3.s1 = nd >= 2 ? s.geom.size[nd - 2] : 0x80000000u;
            s.geo3.d2.set(s.geo3.s2);
            s.geo3.d1.set(s.geo3.s1);
            for (int k = 0; k < n_ops; k++) {
                Op3& o = s.ops3[k];
                o.ptr = s.ops[k].ptr;
                if (s.ops[k].flat) {
                    o.st2 = 1; o.st1 = s.geo3.s2; o.st0 = nd >= 3 ? s.geo3.s2 * s.geo3.s1 : 0;
                } else {
                    o.st2 = (uint32_t)s.ops[k].stride[nd - 1];
                    o.st1 = nd >= 2 ? (uint32_t)s.ops[k].stride[nd - 2] : 0;
                    o.st0 = nd >= 3 ? (uint32_t)s.ops[k].stride[0] : 0;
                }
            }
        }
        if (!emit(s)) return false;
    }
    return true;
}

// True when runs of V elements never straddle an innermost row and every vector access of the
// slab is aligned, so the typed kernel may use its vector path.
inline bool slab_aligned(const Slab& s, int n_ops, const int* op_bytes, int out_bytes, int V) {
    // accesses are at most 16 bytes wide, whatever the run length
    auto need = [V](int bytes) { const size_t run = (size_t)bytes * V; return run < 16 ? run : (size_t)16; };
    if (!aligned_to(s.out, need(out_bytes))) return false;
    for (int k = 0; k < n_ops; k++) if (!aligned_to(s.ops3[k].ptr, need(op_bytes[k]))) return false;
    if (s.geo3.simple) return true;
    if (s.geo3.s2 % (uint32_t)V) return false;
    for (int k = 0; k < n_ops; k++) if ((s.ops3[k].st0 % V) || (s.ops3[k].st1 % V)) {
        if (s.ops3[k].st2 != 0) return false;           // a vector-loaded operand needs aligned rows
    }
    return true;
}

template <class Body>
bool launch_body(const char* name, const Body& body, size_t n) {
    DeviceState* st = acquire_device();
    if (!st) return false;
    // programmatic stream serialisation (see wait_for_previous_kernel); TOPS_PDL=0 switches it off
    static const bool overlap = [] { const char* e = getenv("TOPS_PDL"); return !(e && e[0] == '0'); }();
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(kEwThreads);
    cfg.stream = current_stream();
    cfg.attrs = attr;
    cfg.numAttrs = overlap ? 1 : 0;
    if constexpr (Body::kGroups > 0) {
        const size_t tile = (size_t)32 * Body::kV * Body::kGroups;
        cfg.gridDim = dim3(grid_for(((n + tile - 1) / tile) * 32, kEwThreads, st->sm_count, kEwCtasPerSm));
        check_cuda(cudaLaunchKernelEx(&cfg, ew_kernel_tiled<Body>, body, (uint32_t)n), name);
    } else {
        const size_t runs = (n + Body::kV - 1) / Body::kV;
        cfg.gridDim = dim3(grid_for(runs, kEwThreads, st->sm_count, kEwCtasPerSm));
        check_cuda(cudaLaunchKernelEx(&cfg, ew_kernel<Body>, body, (uint32_t)n), name);
    }
    return TOPS_CHECK_LAUNCH(name);
}

}  // namespace tops
