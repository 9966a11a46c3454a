// Shared device helpers for the sm_100a kernels: mbarrier, 1-D TMA bulk copies,
// programmatic dependent launch, mixed-sign dp4a.  Inline PTX only; no library code.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace terb {

// Device-side error codes written to the handle's status word.
enum : int { DEV_OK = 0, DEV_TIMEOUT_MBAR = 1, DEV_TIMEOUT_FLAG = 2 };

// Upper bound on mbarrier polls.  Each try_wait suspends for a hardware-defined
// interval, so this is of the order of a second before a kernel gives up.
constexpr uint32_t kMbarSpinLimit = 1u << 22;

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
// Make barrier initialisation visible to the async (TMA) proxy.
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
// The same test with a suspend-time hint: the thread may sleep up to `ns` nanoseconds inside the instruction and
// is woken when the phase completes, so a waiting warp stops competing for issue slots with working ones.
__device__ __forceinline__ bool mbar_try_wait_hint(uint64_t* bar, uint32_t parity, uint32_t ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(ns)
        : "memory");
    return ok != 0;
}
// Bounded wait built on it, limited by time (about two seconds) rather than by a poll count, since one poll may
// now take up to the hint.  Same contract as mbar_wait_bounded.
__device__ __forceinline__ bool mbar_wait_sleepy(uint64_t* bar, uint32_t parity, int* status) {
    constexpr uint32_t kHintNs = 20000;
    if (mbar_try_wait_hint(bar, parity, kHintNs)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t0));
    bool expired_elsewhere = false;
    for (uint32_t i = 1;; ++i) {
        if (mbar_try_wait_hint(bar, parity, kHintNs)) return true;
        if ((i & 63u) == 0) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            if (status && *reinterpret_cast<volatile int*>(status) != DEV_OK) { expired_elsewhere = true; break; }
            if (t - t0 > 2000000000ull) break;
        }
    }
    if (status) atomicExch(status, DEV_TIMEOUT_MBAR);
    // Second bounded chance for copies still in flight before the CTA moves on.
    const uint32_t second = expired_elsewhere ? 64u : 50000u;
    for (uint32_t i = 0; i < second; ++i)
        if (mbar_try_wait_hint(bar, parity, kHintNs)) return false;
    return false;
}

// Bounded wait.  On expiry records DEV_TIMEOUT_MBAR in *status and returns false;
// the caller carries on (its results are then meaningless, and the host sees the code).
// Once any wait of the launch has expired (the status word is set), later waits give up after a short
// budget instead of spinning the full limit each: a kernel with one lost copy returns promptly.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, int* status) {
    bool expired_elsewhere = false;
    for (uint32_t i = 0; i < kMbarSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 0x3fffu) == 0x3fffu && status && *reinterpret_cast<volatile int*>(status) != DEV_OK) {
            expired_elsewhere = true;
            break;
        }
    }
    if (status) atomicExch(status, DEV_TIMEOUT_MBAR);
    // Second bounded chance for copies still in flight before the CTA moves on.
    const uint32_t second = expired_elsewhere ? (1u << 14) : kMbarSpinLimit;
    for (uint32_t i = 0; i < second; ++i)
        if (mbar_try_wait(bar, parity)) return false;
    return false;
}

// 1-D TMA bulk copy global -> shared, completion counted on an mbarrier.
// dst, src 16-byte aligned; bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
            smem_u32(dst)),
        "l"(src), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}

// Programmatic dependent launch: let the next kernel in the stream start its
// prologue; wait until the kernels this one depends on have finished and flushed.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// d = c + sum_i s8(a.byte[i]) * u8(b.byte[i])
__device__ __forceinline__ int dp4a_su(int a, uint32_t b, int c) {
    int d;
    asm("dp4a.s32.u32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Packed-trit multiply-accumulate (internal weight layout: field i of every weight byte is column i,
// re-coded to u = trit + 1).
// Accumulates one 32-bit word of weights (4 k x 4 columns) against 4 int8 activations.
// t collects the UNMASKED product  S0 + 4*S1 + 16*S2 + 64*S3  (no AND needed); a1..a3 collect
// 4*S1, 16*S2, 64*S3 from masked words; column 0 is recovered as t - a1 - a2 - a3.
__device__ __forceinline__ void mac16(uint32_t w, int x, int& t, int& a1, int& a2, int& a3) {
    t = dp4a_su(x, w, t);
    a1 = dp4a_su(x, w & 0x0C0C0C0Cu, a1);
    a2 = dp4a_su(x, w & 0x30303030u, a2);
    a3 = dp4a_su(x, w & 0xC0C0C0C0u, a3);
}
__device__ __forceinline__ void mac64(const uint4& w, const int4& xv, int& t, int& a1, int& a2, int& a3) {
    mac16(w.x, xv.x, t, a1, a2, a3);
    mac16(w.y, xv.y, t, a1, a2, a3);
    mac16(w.z, xv.z, t, a1, a2, a3);
    mac16(w.w, xv.w, t, a1, a2, a3);
}

}  // namespace terb
