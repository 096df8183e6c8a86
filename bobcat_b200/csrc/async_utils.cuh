// Device wrappers of the asynchronous machinery of sm_100a used by the prefill kernel: mbarriers,
// bulk (TMA) copies, cp.async, tensor memory and tcgen05 matrix instructions. Shared-memory
// addresses are 32-bit shared::cta integers throughout. Every wait is bounded: it returns false
// when it ran out instead of spinning forever.
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace bc {
namespace k {
namespace async {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
// Make freshly initialised barriers visible to the async proxy (bulk copies, tcgen05.commit).
__device__ __forceinline__ void mbar_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
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
// Wait for the phase of `parity` to complete. Gives up after `limit` polls, or as soon as `*dead`
// (a shared flag another thread of the CTA raised when its own wait ran out) is set.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, uint32_t limit, volatile int* dead) {
    for (uint32_t spin = 0; spin < limit; ++spin) {
        if (mbar_test(bar, parity)) return true;
        if ((spin & 255u) == 255u && *dead) return false;
    }
    return false;
}

// ---- copies

// Bulk copy global -> shared, completing `bytes` on `bar`. Addresses and size multiples of 16.
__device__ __forceinline__ void bulk_load(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes),
                 "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void cp_async_16(uint32_t dst, const void* src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_4(uint32_t dst, const void* src) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// Order this thread's generic-proxy shared-memory writes before later async-proxy reads (tcgen05.mma).
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---- tensor memory and tcgen05

// Whole warp: allocate `columns` (a power of two, at least 32) and write the base address to `slot`.
__device__ __forceinline__ void tmem_alloc(uint32_t slot, uint32_t columns) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot), "r"(columns) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t columns) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(columns) : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor of a K-major operand without swizzle. The operand is made of
// core matrices of 8 rows x 16 bytes (128 contiguous bytes); `k_step` is the byte distance between
// core matrices adjacent along K, `row_step` between groups of 8 rows.
__device__ __forceinline__ uint64_t umma_desc(uint32_t addr, uint32_t k_step, uint32_t row_step) {
    uint64_t d = (uint64_t)((addr & 0x3ffffu) >> 4);
    d |= (uint64_t)(k_step >> 4) << 16;    // leading-dimension byte offset
    d |= (uint64_t)(row_step >> 4) << 32;  // stride-dimension byte offset
    d |= 1ull << 46;                       // descriptor version of sm_100
    return d;
}
// Instruction descriptor of kind::f16: f16 A and B, both K-major, f32 accumulator, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc_f16(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}
// One thread: D[tmem] (+)= A * B^T over K = 16.
__device__ __forceinline__ void umma_f16(uint32_t tmem_d, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}" ::"r"(tmem_d),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// One thread: `bar` gets one arrival when every tcgen05.mma this thread issued so far has finished.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// Whole warp: 16 consecutive accumulator columns of this warp's 32 lanes (lane i of the warp reads
// TMEM lane 32 * (warp % 4) + i); `taddr` carries the lane in bits 16.. and the column below.
__device__ __forceinline__ void tmem_load_16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n\t"
        "tcgen05.wait::ld.sync.aligned;"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

}  // namespace async
}  // namespace k
}  // namespace bc
