// One-shot sum of small fp32 partial outputs across the GPUs of one NVLink/NVSwitch box, done in
// the epilogue of the decode kernels instead of a separate collective launch.
//
// Every rank owns one exchange buffer; every rank maps all buffers (own: plain device pointer,
// peers: CUDA IPC mappings).  A step of the expert-parallel MoE / tensor-parallel dense FFN ends
// like this in each CTA, for the output rows that CTA owns:
//
//   1. store its partial values into slot[parity][own rank] of EVERY rank's buffer (plain peer
//      stores over NVLink; its own buffer included),
//   2. CTA barrier, then one thread: system-scope fence and a release store of step+1 into
//      flag[parity][own rank][cta] of every rank's buffer,
//   3. the same thread waits (bounded) until flag[parity][q][cta] of its OWN buffer equals step+1
//      for every rank q, CTA barrier,
//   4. sum slot[parity][q] over q in rank order from its own buffer (L2 loads), add the residual,
//      round, store.  The order is fixed, so all ranks produce bit-identical outputs.
//
// `step` is a counter kept in the rank's own buffer and advanced by the kernel, so a captured CUDA
// graph can be replayed.  parity = step & 1 alternates between two sets of slots and flags: a rank
// can run at most one step ahead of the slowest one (it needs everyone's contribution to finish a
// step), so two sets are enough to keep a fast rank from overwriting what a slow one still reads.
// All ranks must make the same sequence of calls with the same shapes (same grid, same rows per
// CTA); a rank that never shows up makes the others' waits run out, which sets the status word
// and ends the kernel - nothing spins forever.
//
// Peer memory is touched with plain ld/st instructions only (no bulk copies, no switch reductions).
#pragma once

#include "mk36_common.cuh"

namespace mk36 {

constexpr int kCommMaxRanks = MK36_MAX_RANKS;
constexpr int kCommMaxCtas = 1024;             // flags per (parity, source rank)
constexpr int kCommMaxElems = 8 * 8192;        // fp32 values per (parity, source rank): 8 tokens x hidden <= 8192
constexpr size_t kCommHeaderBytes = 4096;      // step counter
constexpr size_t kCommFlagBytes = (size_t)2 * kCommMaxRanks * kCommMaxCtas * 4;
constexpr size_t kCommSlotBytes = (size_t)2 * kCommMaxRanks * kCommMaxElems * 4;
constexpr size_t kCommBytes = kCommHeaderBytes + kCommFlagBytes + kCommSlotBytes;
constexpr int kStatusCommWait = 401;           // a peer's contribution never arrived
constexpr unsigned long long kCommWaitLimitNs = 1000ull * 1000ull * 1000ull;

// Passed to the kernels by value.  world <= 1 means "no exchange".
struct CommParams {
    int rank = 0;
    int world = 1;
    unsigned char* buf[kCommMaxRanks] = {};
};

// Fills `out` from the C-ABI descriptor (nullptr = single GPU); checks ranks and pointers.
int comm_params_from(const mk36_comm* c, int hidden, CommParams* out, const char* what);

#if defined(__CUDACC__)

// Buffer of rank q.  Written as selects over constant indices: indexing the kernel-parameter array with
// a run-time value would make the compiler copy the whole parameter block to local memory.
__device__ __forceinline__ unsigned char* comm_buf(const CommParams& c, int q) {
    unsigned char* r = c.buf[0];
#pragma unroll
    for (int i = 1; i < kCommMaxRanks; ++i)
        if (q == i) r = c.buf[i];
    return r;
}

__device__ __forceinline__ unsigned* comm_step_ptr(unsigned char* base) { return reinterpret_cast<unsigned*>(base); }

__device__ __forceinline__ unsigned* comm_flag(unsigned char* base, int parity, int src, int cta) {
    return reinterpret_cast<unsigned*>(base + kCommHeaderBytes) + ((size_t)(parity * kCommMaxRanks + src) * kCommMaxCtas + cta);
}

__device__ __forceinline__ float* comm_slot(unsigned char* base, int parity, int src) {
    return reinterpret_cast<float*>(base + kCommHeaderBytes + kCommFlagBytes) + (size_t)(parity * kCommMaxRanks + src) * kCommMaxElems;
}

__device__ __forceinline__ unsigned comm_read_step(const CommParams& c) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(comm_step_ptr(comm_buf(c, c.rank))) : "memory");
    return v;
}

__device__ __forceinline__ void comm_write_step(const CommParams& c, unsigned v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(comm_step_ptr(comm_buf(c, c.rank))), "r"(v) : "memory");
}

// One thread, after a CTA-wide barrier that follows the partial stores of the whole CTA.
__device__ __forceinline__ void comm_signal(const CommParams& c, int parity, int cta, unsigned value) {
    asm volatile("fence.acq_rel.sys;" ::: "memory");
    for (int q = 0; q < c.world; ++q) {
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(comm_flag(comm_buf(c, q), parity, c.rank, cta)), "r"(value) : "memory");
    }
}

// One thread.  Returns false (and records the status code) when a contribution does not arrive
// within the limit.
static __device__ __noinline__ bool comm_wait_on(unsigned char* own, int world, Control* ctl, int parity, int cta, unsigned value) {
    const unsigned long long t0 = global_timer_ns();
    for (int q = 0; q < world; ++q) {
        const unsigned* f = comm_flag(own, parity, q, cta);
        unsigned spins = 0;
        for (;;) {
            unsigned v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(f) : "memory");
            if (v == value) break;
            if ((++spins & 63u) == 0u && global_timer_ns() - t0 > kCommWaitLimitNs) {
                atomicCAS(&ctl->status, 0, kStatusCommWait);
                return false;
            }
        }
    }
    return true;
}

// (The out-of-line part takes plain values: a reference to the kernel parameters would force a copy of
// the parameter block into local memory.)
__device__ __forceinline__ bool comm_wait(const CommParams& c, Control* ctl, int parity, int cta, unsigned value) {
    return comm_wait_on(comm_buf(c, c.rank), c.world, ctl, parity, cta, value);
}

// Sum over the ranks, in rank order, of element `idx` of this step's slots in the own buffer.
__device__ __forceinline__ float comm_sum(const CommParams& c, int parity, size_t idx) {
    float v = 0.0f;
    unsigned char* own = comm_buf(c, c.rank);
    for (int q = 0; q < c.world; ++q) v += __ldcg(comm_slot(own, parity, q) + idx);
    return v;
}

#endif  // __CUDACC__

}  // namespace mk36
