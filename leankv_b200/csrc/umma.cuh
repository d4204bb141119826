// Fifth-generation tensor core (tcgen05) helpers shared by the kernels that run 128 x 128 x K products
// with operands in shared memory and fp32 accumulators in tensor memory.
//
// Operand layout (K-major, no swizzle): element (row, k) of a 128-row fp16 operand with K = 128 lives at
//   (row / 8) * kSbo + (k / 8) * kLbo + (row % 8) * 16 + (k % 8) * 2   bytes,
// i.e. 8 x 8 core matrices of 128 contiguous bytes, the 16 core matrices of a row group side by side. A
// shared-memory descriptor names the start of such an operand; one tcgen05.mma (K = 16) consumes two core
// matrices along K, so k-step ks starts 2 * kLbo * ks bytes further.
#pragma once

#include <stdint.h>

namespace leankv {
namespace umma {

constexpr int kRows = 128;                           // M and N of the product
constexpr int kK = 128;                              // full K of an operand tile
constexpr uint32_t kLbo = 128;                       // next core matrix along K
constexpr uint32_t kSbo = (kK / 8) * 128;            // next group of 8 rows: 2048 bytes
constexpr uint32_t kTileBytes = kRows * kK * 2;      // one 128 x 128 fp16 operand: 32 KB
constexpr uint32_t kTmemCols = 128;                  // fp32 accumulator: 128 lanes x 128 columns
// instruction descriptor: D fp32 (bits 4-5 = 1), A and B fp16 (0), both K-major (bits 15, 16 = 0), N / 8 at bit 17,
// M / 16 at bit 24
constexpr uint32_t kIdesc = (1u << 4) | ((uint32_t)(kRows / 8) << 17) | ((uint32_t)(kRows / 16) << 24);
constexpr int kWaitLimit = 1 << 20;

__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t desc(uint32_t addr) {
    // start address >> 4 (14 bits), leading byte offset >> 4 at bit 16, stride byte offset >> 4 at bit 32,
    // descriptor version 1 at bit 46, no swizzle (layout type 0 at bit 61)
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(kLbo >> 4) << 16) | ((uint64_t)(kSbo >> 4) << 32) |
           (1ull << 46);
}
__device__ __forceinline__ uint32_t offset(int row, int k8) {     // byte offset of the 16-byte piece (row, 8 k8 ..)
    return (uint32_t)(row >> 3) * kSbo + (uint32_t)k8 * kLbo + (uint32_t)(row & 7) * 16;
}
// D[128 x 128] (+)= A[128 x 16] . B[128 x 16]^T; issued by one thread
__device__ __forceinline__ void mma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(kIdesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// the mbarrier is arrived on once every MMA issued so far by this thread has completed
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// one warp (all 32 lanes) allocates / frees kTmemCols columns; the base address lands in *slot (shared memory)
__device__ __forceinline__ void tmem_alloc(uint32_t slot_addr) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(kTmemCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free(uint32_t tmem_base) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// operands written through the generic proxy become visible to the tensor core's async proxy
__device__ __forceinline__ void fence_operands() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// 32 consecutive accumulator columns of this thread's lane (lane = lane0 + lane id; lane0 = 32 * (warp % 4))
__device__ __forceinline__ void ld32(uint32_t (&r)[32], uint32_t tmem_base, int lane0, int col0) {
    const uint32_t taddr = tmem_base + ((uint32_t)lane0 << 16) + (uint32_t)col0;
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ---- the same with explicit tile geometry (operands whose K extent is not 128, N other than 128) ----
// K-major blocked operand with `k_chunks` 16-byte pieces per row: core matrices of a row group side by side
// (leading byte offset 128), row groups k_chunks * 128 bytes apart.
__device__ __forceinline__ uint64_t desc_k(uint32_t addr, int k_chunks) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(kLbo >> 4) << 16) |
           ((uint64_t)(((uint32_t)k_chunks * 128u) >> 4) << 32) | (1ull << 46);
}
__device__ __forceinline__ uint32_t offset_k(int row, int k8, int k_chunks) {
    return (uint32_t)(row >> 3) * (uint32_t)k_chunks * 128u + (uint32_t)k8 * kLbo + (uint32_t)(row & 7) * 16;
}
// instruction descriptor for D fp32 = A fp16 . B fp16, both K-major, M = 128, N = n
__host__ __device__ constexpr uint32_t idesc_n(int n) { return (1u << 4) | ((uint32_t)(n / 8) << 17) | ((uint32_t)(kRows / 16) << 24); }
__device__ __forceinline__ void mma_f16_n(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void tmem_alloc_n(uint32_t slot_addr, uint32_t n_cols) {      // n_cols: power of two >= 32
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_addr), "r"(n_cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_free_n(uint32_t tmem_base, uint32_t n_cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(n_cols) : "memory");
}
// 32 consecutive accumulator columns of this thread's lane, written back
__device__ __forceinline__ void st32(const uint32_t (&r)[32], uint32_t tmem_base, int lane0, int col0) {
    const uint32_t taddr = tmem_base + ((uint32_t)lane0 << 16) + (uint32_t)col0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// the same product with the A operand in tensor memory: lane = row, two fp16 per 32-bit column (element 2c in the
// low half), so a K = 16 step reads 8 columns starting at tmem_a
__device__ __forceinline__ void mma_f16_ts(uint32_t tmem_d, uint32_t tmem_a, uint64_t b_desc, uint32_t idesc,
                                           uint32_t accumulate) {
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t"
        "}\n"
        :
        : "r"(tmem_d), "r"(tmem_a), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
// 16 consecutive columns of this thread's lane, written
__device__ __forceinline__ void st16(const uint32_t (&r)[16], uint32_t tmem_base, int lane0, int col0) {
    const uint32_t taddr = tmem_base + ((uint32_t)lane0 << 16) + (uint32_t)col0;
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}
// one arrival on an mbarrier whose phase completes after a fixed number of them
__device__ __forceinline__ void bar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void bar_init_n(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void bar_init(uint32_t bar) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(bar));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// bounded wait for the given phase parity: false if it did not complete within kWaitLimit polls
__device__ __forceinline__ bool bar_wait(uint32_t bar, uint32_t parity) {
    for (int i = 0; i < kWaitLimit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}

}  // namespace umma
}  // namespace leankv
