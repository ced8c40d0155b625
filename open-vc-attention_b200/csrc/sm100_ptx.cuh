// Thin inline-PTX wrappers for sm_100a: mbarrier, TMA tile loads, tensor memory and tcgen05 MMA.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace ovc {
namespace ptx {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity)
        : "memory");
    return done != 0;
}
// Same test, but the hardware may suspend the thread for up to `hint_ns` while the phase is pending,
// so a waiting warp does not burn issue slots.
__device__ __forceinline__ bool mbar_try_wait_sleep(uint32_t bar, uint32_t parity, uint32_t hint_ns) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(bar), "r"(parity), "r"(hint_ns)
        : "memory");
    return done != 0;
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA: 4-D tiled load, global -> shared, completion on an mbarrier -----------------------
__device__ __forceinline__ void tma_load_4d(uint32_t dst, const void* tmap, uint32_t bar, int c0, int c1, int c2,
                                            int c3, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint"
        " [%0], [%1, {%3, %4, %5, %6}], [%2], %7;"
        :
        : "r"(dst), "l"(tmap), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const void* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ uint64_t policy_evict_last() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}

// ---- tensor memory -------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t result_smem, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(result_smem), "r"(columns)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t* r) {
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
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]),
          "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]),
          "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ uint32_t tmem_ld1(uint32_t taddr) {
    uint32_t r;
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x1.b32 {%0}, [%1];" : "=r"(r) : "r"(taddr) : "memory");
    return r;
}
__device__ __forceinline__ void tmem_st1(uint32_t taddr, uint32_t r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(taddr), "r"(r) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t* r) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* r) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        :
        : "r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const uint32_t* r) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"r"(taddr), "r"(r[0]),
                 "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7])
                 : "memory");
}

// ---- tcgen05 MMA, FP8 E4M3 x E4M3 -> FP32, one CTA -------------------------------------------
// Four K-steps of one 128-wide MMA, issued by one elected lane while the whole warp executes the
// (convergent) code, so that descriptors and addresses stay warp-uniform values.  `a_lo` / `b_lo` are
// the low words of shared-memory matrix descriptors: K-major rows of 128 bytes in the 128-byte swizzle,
// 8-row groups 1024 bytes apart (tile base 1024-byte aligned), high word kSmemDescHi; K advances 32 bytes
// (2 in descriptor units) per step.
constexpr uint32_t kSmemDescHi = (1024u >> 4) | (1u << 14) | (2u << 29);
__device__ __forceinline__ uint32_t smem_desc_lo(uint32_t saddr) { return ((saddr & 0x3FFFFu) >> 4) | (1u << 16); }

__device__ __forceinline__ void mma4_f8_ss(uint32_t d_tmem, uint32_t a_lo, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred leader;\n\t.reg .b64 da, db;\n\t.reg .b32 al, bl;\n\t"
        "elect.sync _|leader, 0xFFFFFFFF;\n\t"
        "mov.b64 da, {%1, %3};\n\tmov.b64 db, {%2, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, 0;\n\t"
        "add.u32 al, %1, 2;\n\tadd.u32 bl, %2, 2;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, 1;\n\t"
        "add.u32 al, %1, 4;\n\tadd.u32 bl, %2, 4;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, 1;\n\t"
        "add.u32 al, %1, 6;\n\tadd.u32 bl, %2, 6;\n\tmov.b64 da, {al, %3};\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], da, db, %4, 1;\n\t}"
        :
        : "r"(d_tmem), "r"(a_lo), "r"(b_lo), "r"(kSmemDescHi), "r"(idesc)
        : "memory");
}
// Same with A in tensor memory (8 columns per K-step); `accumulate_first` = 0 starts a new accumulation.
__device__ __forceinline__ void mma4_f8_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                           uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred leader, p;\n\t.reg .b64 db;\n\t.reg .b32 bl, ta;\n\t"
        "elect.sync _|leader, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t"
        "add.u32 bl, %2, 2;\n\tadd.u32 ta, %1, 8;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t"
        "add.u32 bl, %2, 4;\n\tadd.u32 ta, %1, 16;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t"
        "add.u32 bl, %2, 6;\n\tadd.u32 ta, %1, 24;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kSmemDescHi), "r"(idesc), "r"(accumulate_first)
        : "memory");
}
// The same product with B in its MN-major form (rows of the shared-memory tile are the K index, 128 bytes of N per
// row, 8-row groups 1024 bytes apart): a K-step of 32 rows advances the descriptor by 4 x 1024 bytes, and N beyond
// the first 128 bytes continues `lbo` bytes after the tile (the leading-dimension offset in `b_lo`, bits 16-29).
__device__ __forceinline__ void mma4_f8_ts_bmn(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc,
                                               uint32_t accumulate_first) {
    asm volatile(
        "{\n\t.reg .pred leader, p;\n\t.reg .b64 db;\n\t.reg .b32 bl, ta;\n\t"
        "elect.sync _|leader, 0xFFFFFFFF;\n\t"
        "setp.ne.b32 p, %5, 0;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [%1], db, %4, p;\n\t"
        "add.u32 bl, %2, 256;\n\tadd.u32 ta, %1, 8;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t"
        "add.u32 bl, %2, 512;\n\tadd.u32 ta, %1, 16;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t"
        "add.u32 bl, %2, 768;\n\tadd.u32 ta, %1, 24;\n\tmov.b64 db, {bl, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], [ta], db, %4, 1;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kSmemDescHi), "r"(idesc), "r"(accumulate_first)
        : "memory");
}
__device__ __forceinline__ uint32_t smem_desc_lo_bmn(uint32_t saddr, uint32_t lbo_bytes) {
    return ((saddr & 0x3FFFFu) >> 4) | ((lbo_bytes >> 4) << 16);
}
// One BF16 x BF16 -> FP32 product of depth 16 added to the accumulator: A = 8 columns of tensor memory (two
// BF16 values per column), B = 32 bytes of each 128-byte row of a swizzled shared-memory tile.
__device__ __forceinline__ void mma_bf16_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred leader;\n\t.reg .b64 db;\n\t"
        "elect.sync _|leader, 0xFFFFFFFF;\n\t"
        "mov.b64 db, {%2, %3};\n\t"
        "@leader tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], db, %4, 1;\n\t}"
        :
        : "r"(d_tmem), "r"(a_tmem), "r"(b_lo), "r"(kSmemDescHi), "r"(idesc)
        : "memory");
}
__device__ __forceinline__ void mma_commit_elect(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred leader;\n\t"
        "elect.sync _|leader, 0xFFFFFFFF;\n\t"
        "@leader tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar)
        : "memory");
}

// Instruction descriptor for kind::f8f6f4, E4M3 x E4M3 -> F32, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_e4m3_f32(int n) {
    return (1u << 4)                              // accumulator format F32
           | (0u << 7) | (0u << 10)               // A, B format E4M3
           | (0u << 15) | (0u << 16)              // A, B K-major
           | (static_cast<uint32_t>(n >> 3) << 17)  // N / 8
           | (static_cast<uint32_t>(128 >> 4) << 24);  // M / 16
}

// The same with B MN-major (bit 16).
__host__ __device__ constexpr uint32_t idesc_e4m3_f32_bmn(int n) { return idesc_e4m3_f32(n) | (1u << 16); }

// Instruction descriptor for kind::f16, BF16 x BF16 -> F32, both operands K-major, M = 128.
__host__ __device__ constexpr uint32_t idesc_bf16_f32(int n) {
    return (1u << 4)                              // accumulator format F32
           | (1u << 7) | (1u << 10)               // A, B format BF16
           | (0u << 15) | (0u << 16)              // A, B K-major
           | (static_cast<uint32_t>(n >> 3) << 17)  // N / 8
           | (static_cast<uint32_t>(128 >> 4) << 24);  // M / 16
}

}  // namespace ptx
}  // namespace ovc
