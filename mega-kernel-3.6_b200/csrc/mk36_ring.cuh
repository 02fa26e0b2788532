// Shared-memory ring fed by the bulk-copy engine (TMA, 1-D cp.async.bulk into the issuing CTA only) and
// drained by compute warps: mbarrier wrappers with bounded waits, and the copy itself.
//
// A stage is a fixed-size slot of shared memory with two mbarriers: `full` (armed by the producer
// with the byte count of the copy it issues, completed by the copy engine) and `empty` (one
// arrival per consumer warp that has finished reading the slot).  Chunk n of a CTA's stream lives
// in stage n % depth; its barrier phase parity is (n / depth) & 1.
//
// Every wait is bounded: when it runs out, or when another warp of the CTA has already given up
// (abort flag in shared memory), it returns false, the caller records a status code in the
// workspace and the CTA drains and leaves instead of hanging.
#pragma once

#include "mk36_common.cuh"

namespace mk36 {

#if defined(__CUDACC__)

__device__ __forceinline__ unsigned smem_addr(const void* p) {
    return static_cast<unsigned>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(count) : "memory");
}

// Makes freshly initialised barriers visible to the copy engine; follow with a CTA-wide sync.
__device__ __forceinline__ void mbar_init_fence() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(unsigned long long* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_addr(bar)) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(unsigned long long* bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(unsigned long long* bar, unsigned parity) {
    unsigned done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}"
        : "=r"(done)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Bounded wait for the phase with the given parity.  `abort_flag` is a shared-memory word that
// any warp of the CTA sets when it gives up.  The spinning part is kept out of line: these
// kernels run every code path about once per launch, so their time is sensitive to code size.
static __device__ __noinline__ bool mbar_wait_slow(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                           unsigned long long limit_ns) {
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (!mbar_try_wait(bar, parity)) {
        if ((++spins & 31u) == 0u) {
            if (*abort_flag != 0) return false;
            if (global_timer_ns() - t0 > limit_ns) {
                *abort_flag = 1;
                return false;
            }
        }
    }
    return true;
}

__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity, volatile int* abort_flag,
                                          unsigned long long limit_ns = kWaitLimitNs) {
    if (mbar_try_wait(bar, parity)) return true;
    return mbar_wait_slow(bar, parity, abort_flag, limit_ns);
}

// Bulk copy global -> shared of `bytes` (multiple of 16, both addresses 16-byte aligned); completes
// `bytes` transaction bytes on `bar`.  The destination is this CTA's own shared memory.
__device__ __forceinline__ void bulk_copy_g2s(void* dst_smem, const void* src_gmem, unsigned bytes, unsigned long long* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_addr(dst_smem)),
                 "l"(src_gmem), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

// Asks the memory system to bring `bytes` starting at `src` into L2 (no destination, no barrier).
__device__ __forceinline__ void bulk_prefetch_l2(const void* src_gmem, unsigned bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src_gmem), "r"(bytes) : "memory");
}

// Barrier among a subset of the CTA's warps (id 1..15, `threads` a multiple of 32).
__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

__device__ __forceinline__ uint4 lds128(const void* p) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(smem_addr(p)));
    return v;
}

#endif  // __CUDACC__

}  // namespace mk36
