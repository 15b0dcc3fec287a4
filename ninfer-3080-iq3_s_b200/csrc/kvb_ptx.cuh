// kvb_ptx.cuh -- thin wrappers over the sm_100a PTX the attention kernels use: mbarriers, bulk async
// copies (TMA engine, no multicast anywhere), warp-level tensor-core MMA, and nibble -> fp16 unpacking.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>

namespace kvb {

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// One arrival of the calling thread (release at CTA scope: its earlier shared-memory writes are visible to a waiter).
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
constexpr uint32_t kWaitHintNs = 2000;  // upper bound of one probe's hardware suspend time
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kWaitHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait of a whole warp: gives up after kSpinLimit probes (each suspends for at most kWaitHintNs,
// about one second in total) and reports failure instead of spinning forever.  The verdict is made
// warp-uniform so that callers can branch on it and still use full-mask warp primitives afterwards.
constexpr uint32_t kSpinLimit = 1u << 19;
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity) {
    bool ok = false;
    for (uint32_t i = 0; i < kSpinLimit && !ok; ++i) ok = mbar_try_wait(bar, parity);
    return __all_sync(0xffffffffu, ok);
}

// The same wait for lanes that may have diverged (some found the barrier complete at their first probe): no vote.
// Every lane probes the same barrier phase, so a lane can run out of probes only if no lane ever saw it complete.
__device__ __forceinline__ bool mbar_wait_lane_bounded(uint64_t* bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; ++i)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}

// Generic-proxy accesses to shared memory made before this fence are ordered before later async-proxy
// (bulk copy) accesses: needed before a buffer that was read with ld.shared is refilled by a bulk copy.
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// Bulk async copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned),
// completion counted on `bar`.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst)),
                 "l"(src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// D(16x8, f32) += A(16x16, f16, row) * B(16x8, f16, col)
__device__ __forceinline__ void mma16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                         uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch.  A kernel launched with the programmatic-stream-serialization attribute may
// start while its predecessor in the stream still runs (as soon as every CTA of the predecessor has called
// launch_dependents or exited); it must call grid_dependency_wait() before touching anything the predecessor
// writes: that returns when the predecessor has completed and its memory is visible.  Both are no-ops in a
// kernel launched the ordinary way.
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// Barrier `id` (1..15; 0 is __syncthreads) among `threads` threads (a multiple of 32): whole warps arrive and wait.
__device__ __forceinline__ void named_barrier_sync(int id, int threads) {
    asm volatile("barrier.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ uint32_t lop3_and_or(uint32_t x, uint32_t mask, uint32_t orv) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(x), "r"(mask), "r"(orv));  // (x & mask) | orv
    return r;
}
__device__ __forceinline__ uint32_t hsub2_u32(uint32_t a, uint32_t b) {
    uint32_t r;
    asm("sub.f16x2 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(b));
    return r;
}

// Eight 4-bit codes of one 32-bit word -> four half2 registers, exact:
//   out[0] = (n0, n4)  out[1] = (n1, n5)  out[2] = (n2, n6)  out[3] = (n3, n7)     (low half, high half)
// A nibble at bits 0..3 OR-ed under exponent 2^10 reads as 1024 + n; one at bits 4..7 under 2^6 reads as
// 64 + n; subtracting the bias is exact in fp16.
__device__ __forceinline__ void unpack8(uint32_t w, uint32_t (&out)[4]) {
    const uint32_t w8 = w >> 8;
    out[0] = hsub2_u32(lop3_and_or(w, 0x000F000Fu, 0x64006400u), 0x64006400u);
    out[1] = hsub2_u32(lop3_and_or(w, 0x00F000F0u, 0x54005400u), 0x54005400u);
    out[2] = hsub2_u32(lop3_and_or(w8, 0x000F000Fu, 0x64006400u), 0x64006400u);
    out[3] = hsub2_u32(lop3_and_or(w8, 0x00F000F0u, 0x54005400u), 0x54005400u);
}

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    const __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<const uint32_t*>(&h);
}
__device__ __forceinline__ float2 unpack_half2(uint32_t u) {
    return __half22float2(*reinterpret_cast<const __half2*>(&u));
}

__device__ __forceinline__ float fast_exp2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}

}  // namespace kvb
