// Pieces shared by the kernels that stream weights through a shared-memory ring filled by bulk
// asynchronous copies (cp.async.bulk + mbarrier transaction counts): barrier helpers with BOUNDED
// waits, the bulk-copy instruction, and the f16 decode of E2M1 weights.
#pragma once
#include <cuda_fp16.h>

#include "common.cuh"

namespace smoe {
namespace ring {

__device__ __forceinline__ uint32_t smem_addr(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}
// Bounded wait: false when the phase did not complete within the limit (about two seconds) or
// another role of the CTA raised the abort flag.  The suspend-time hint parks the thread between
// polls, so waiting warps do not take issue slots from working ones.
constexpr uint32_t kSpinLimit = 1u << 19;
constexpr uint32_t kWaitHintNs = 4096;
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const volatile uint32_t* abort_flag) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n selp.u32 %0, 1, 0, p;\n}"
            : "=r"(done)
            : "r"(addr), "r"(parity), "r"(kWaitHintNs)
            : "memory");
        if (done) return true;
        if ((spin & 63u) == 63u && *abort_flag) return false;
    }
    return false;
}
// The same wait by plain polling (no suspend hint): for latency-critical kernels whose whole run is a few
// microseconds -- a parked thread was seen to resume microseconds after its barrier completed.
__device__ __forceinline__ bool mbar_wait_poll(uint64_t* bar, uint32_t parity, const volatile uint32_t* abort_flag) {
    const uint32_t addr = smem_addr(bar);
    for (uint32_t spin = 0; spin < (1u << 24); ++spin) {
        uint32_t done;
        asm volatile("{\n .reg .pred p;\n mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                     : "=r"(done)
                     : "r"(addr), "r"(parity)
                     : "memory");
        if (done) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    return false;
}
// One poll, no suspend: used to drain copies still in flight when a CTA gives up.
__device__ __forceinline__ bool mbar_test(uint64_t* bar, uint32_t parity) {
    uint32_t done;
    asm volatile("{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.u32 %0, 1, 0, p;\n}"
                 : "=r"(done)
                 : "r"(smem_addr(bar)), "r"(parity)
                 : "memory");
    return done != 0;
}
// Contiguous global -> shared copy by the copy engine; completion is counted in bytes on `bar`.
// Both addresses 16-byte aligned, bytes a multiple of 16.  The destination is this CTA's own
// shared memory (a CTA launched without a cluster is a cluster of one); the source is this GPU's
// memory and the copy has a single destination.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

__device__ __forceinline__ void mma_f16(float c[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// the same MMA with a zero addend: starts a fresh partial sum without four register moves
__device__ __forceinline__ void mma_f16_zero(float d[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                             uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}
// 8 E2M1 nibbles (one 32-bit word, nibble q = column q) -> r[b] = f16x2 {column 2b, column 2b+1}, exact
__device__ __forceinline__ void e2m1x8(uint32_t w, uint32_t r[4]) {
    asm("{\n .reg .b8 b0, b1, b2, b3;\n mov.b32 {b0, b1, b2, b3}, %4;\n"
        " cvt.rn.f16x2.e2m1x2 %0, b0;\n cvt.rn.f16x2.e2m1x2 %1, b1;\n"
        " cvt.rn.f16x2.e2m1x2 %2, b2;\n cvt.rn.f16x2.e2m1x2 %3, b3;\n}"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
        : "r"(w));
}
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    uint32_t d;
    asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(d) : "r"(a), "r"(b));
    return d;
}

}  // namespace ring
}  // namespace smoe
