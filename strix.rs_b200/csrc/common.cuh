// Shared device helpers: f16 widening, bounded mbarrier waits, bulk async copies.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace strix {

// Bits of the device status word (one per accelerator, in global memory).
enum : uint32_t {
    STATUS_OK = 0,
    STATUS_WAIT_TIMEOUT = 1u << 0,  // a bounded mbarrier wait ran out
    STATUS_BAD_ARGS = 1u << 1,      // a kernel saw an impossible launch shape
};

// Exact IEEE binary16 -> binary32 widening, subnormals included
// (half::f16::to_f32 as used at crates/strix-models/src/ggml_quant.rs:186-188).
__device__ __forceinline__ float f16_bits_to_f32(uint16_t h) {
    return __half2float(__ushort_as_half(h));
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// Wait for a phase with an iteration limit. On expiry the caller's status word
// gets STATUS_WAIT_TIMEOUT and the function returns false; the kernel carries on
// to its exit without touching the data, so nothing spins for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity, uint32_t *status) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
    return false;
}

// A wait that polls without ever suspending (mbarrier.test_wait): for the few threads of a kernel whose
// reaction time IS its throughput (the hand-over of a TMEM accumulator between the MMA issuer and the
// warps that drain it). try_wait may park the thread for a system-dependent time when the phase is
// not complete yet, and being woken from that takes longer than the work between two hand-overs.
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t *bar, uint32_t parity, uint32_t *status) {
    for (uint32_t it = 0; it < (1u << 24); ++it) {
        if (mbar_test_wait(bar, parity)) return true;
    }
    if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
    return false;
}

// The same wait for code that shares its SM's issue slots with working warps: each try lets the hardware
// suspend the thread for up to `hint_ns` before it answers, so a waiting warp issues a handful of
// instructions per microsecond instead of spinning. Bounded like mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait_suspended(uint64_t *bar, uint32_t parity, uint32_t *status, uint32_t hint_ns) {
    for (uint32_t it = 0; it < (1u << 22); ++it) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.b32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity), "r"(hint_ns)
            : "memory");
        if (ok) return true;
    }
    if (status) atomicOr(status, STATUS_WAIT_TIMEOUT);
    return false;
}

// 1-D bulk async copy global -> shared, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16. No multicast.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// dp4a with unsigned a (packed u8) and signed b (packed s8).
__device__ __forceinline__ int dp4a_us(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_ss(uint32_t a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

}  // namespace strix
