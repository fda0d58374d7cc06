// Blackwell (sm_100a) building blocks for the tensor-core kernels: mbarrier with BOUNDED waits,
// TMA tile loads, tcgen05 MMA / commit / TMEM load, and the two descriptor encodings.
//
// Every wait in this file gives up after a clock budget and reports through a status word, so a
// kernel built from it returns (with an error flag) instead of spinning forever.
#pragma once

#include <cuda.h>          // CUtensorMap (types only; the encode function is fetched at run time)
#include "common.cuh"

namespace tops {
namespace umma {

constexpr long long kWaitBudgetCycles = 4000000000ll;   // about two seconds at 2 GHz

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier ---------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// One attempt: returns at once when the phase is complete; otherwise the thread may be SUSPENDED until it completes or
// until the time hint runs out (nanoseconds) -- a suspended warp issues nothing, where a short system-chosen limit makes
// every waiting warp a polling loop that shares its scheduler's issue slots with the warps that have work.
constexpr uint32_t kSuspendHintNs = 200000u;
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs) : "memory");
    return ok != 0;
}
// Waits for the phase with the given parity.  Returns false when the budget ran out or another
// role already raised `*abort_flag` (shared memory); the caller then leaves its loop.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, volatile int* abort_flag, long long budget_cycles = kWaitBudgetCycles) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
        #pragma unroll 1
        for (int i = 0; i < 8; i++) if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > budget_cycles) { *abort_flag = 1; return false; }
    }
}

// ---- TMA (each CTA loads its own tiles) ------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}
// Untiled bulk copy global -> shared (both addresses 16-byte aligned, size a multiple of 16 bytes).
__device__ __forceinline__ void bulk_load_1d(void* smem, const void* gmem, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(gmem)), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// Orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy ones.
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tma_load_2d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_load_4d(void* smem, const CUtensorMap* map, uint64_t* bar, int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem)), "l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}

// Tile stores shared -> global (bulk async group of the issuing thread).  The shared-memory source must have been
// made visible to the async proxy (fence_proxy_async_smem after the generic-proxy writes) and must not be
// overwritten until bulk_wait_read says the copy engine has read it.
__device__ __forceinline__ void tma_store_2d(const CUtensorMap* map, const void* smem, int c0, int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(smem_u32(smem)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// All of this thread's committed bulk stores have finished READING shared memory (the buffers may be reused).
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
// All of this thread's committed bulk stores have completed.
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One 32-byte store per thread (address 32-byte aligned): a whole sector in one instruction.
template <int N> __device__ __forceinline__ void store_global_32B(void* ptr, const uint32_t (&w)[N]) {
    static_assert(N >= 8, "eight words");
    asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                 ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]), "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7]) : "memory");
}

// ---- tcgen05 ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t columns) {     // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {        // the same warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync()  { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// D[tmem] (+)= A[smem] * B[smem]; kind f16 covers fp16 / bf16 inputs, f8f6f4 the 8-bit floats.
template <bool FP8>
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t desc_a, uint64_t desc_b, uint32_t idesc, uint32_t accumulate) {
    if constexpr (FP8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(tmem_d), "l"(desc_a), "l"(desc_b), "r"(idesc), "r"(accumulate) : "memory");
    }
}
// The barrier receives one arrival once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_load_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns.
__device__ __forceinline__ void tmem_load_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}
template <int W> __device__ __forceinline__ void tmem_load_chunk(uint32_t taddr, uint32_t (&r)[W]) {
    if constexpr (W == 32) tmem_load_32x32(taddr, r);
    else tmem_load_32x16(taddr, r);
}
__device__ __forceinline__ void tmem_load_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// ---- descriptors ----------------------------------------------------------------------------------------------
// Shared-memory matrix descriptor for a K-major tile whose rows are 128 bytes and which was
// written by TMA with the 128-byte swizzle: 8-row groups are 1024 bytes apart (stride byte
// offset), version field 1, layout type 2 (128-byte swizzle).  The tile base is 1024-aligned.
__device__ __forceinline__ uint64_t smem_desc_k_major_sw128(const void* tile) {
    const uint64_t addr = (uint64_t)(smem_u32(tile) & 0x3FFFFu) >> 4;
    return addr | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, both operands K-major, dense.
// format codes: kind f16 -> 0 fp16, 1 bf16; kind f8f6f4 -> 0 e4m3, 1 e5m2.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t a_format, uint32_t b_format, uint32_t m, uint32_t n) {
    return (1u << 4) | (a_format << 7) | (b_format << 10) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// Byte offset of 16-byte chunk `chunk` of row `row` inside a box whose rows are ROW_BYTES (32 or 64) wide, as the
// copy engine lays it out with the swizzle of that width: the chunk index is XORed with address bits 7 and up
// (one bit for 32-byte rows, two for 64-byte rows).  The box base must be aligned to 1024 bytes.
template <int ROW_BYTES>
__device__ __forceinline__ uint32_t swizzled_chunk(uint32_t row, uint32_t chunk) {
    static_assert(ROW_BYTES == 32 || ROW_BYTES == 64, "row width");
    const uint32_t linear = row * ROW_BYTES;
    const uint32_t mask = ROW_BYTES == 64 ? 3u : 1u;
    return linear + ((chunk ^ ((linear >> 7) & mask)) << 4);
}

}  // namespace umma

// Host: encode a tiled tensor map (rank <= 4) with the 128-byte swizzle and zero fill.
// dims / strides innermost first; strides[0] is implied (element size).  Returns false on error.
bool make_tensor_map(CUtensorMap* out, const void* base, int elem_bytes, bool is_fp8, bool is_fp16, int rank,
                     const uint64_t* dims, const uint64_t* strides_bytes, const uint32_t* box,
                     const uint32_t* elem_strides);
// Host: a row-major matrix [rows][cols] of float32 (elem_bytes 4) or 16-bit (elem_bytes 2) elements seen as boxes of
// box_rows x box_cols whose rows are 32 or 64 bytes wide; the shared-memory image uses the swizzle of that width
// (16-byte chunk index XOR address bits 7.., see swizzled_chunk).
bool make_row_box_map(CUtensorMap* out, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows, uint32_t box_cols);

}  // namespace tops
