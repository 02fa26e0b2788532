// One-shot sum of small fp32 partial outputs across the GPUs of one NVLink/NVSwitch box, done in
// the epilogue of the decode kernels instead of a separate collective launch.
//
// Every rank owns one exchange buffer; every rank maps all buffers (own: plain device pointer,
// peers: CUDA IPC mappings).  A partial value travels together with the number of the step it
// belongs to, as one aligned 64-bit word {value, step + 1}: a 64-bit store is a single access, so
// whoever reads the word sees either the old pair or the new pair, never a mix, and the word is
// its own "ready" flag.  No fence, no separate flag and no barrier is needed, and the cost of the
// exchange is one NVLink store latency.  Per output element o of the rows a CTA owns:
//
//   put:  store {v, step + 1} into slot[parity][own rank][o] of EVERY rank's buffer (own included);
//   get:  for q = 0 .. world-1, in rank order: poll slot[parity][q][o] of the OWN buffer until its
//         tag is step + 1 (bounded), add the value.  Then residual, rounding, store.
//
// The order of the sum is fixed, so all ranks produce bit-identical outputs.
//
// `step` is a counter kept in the rank's own buffer and advanced by the kernel, so a captured CUDA
// graph can be replayed.  parity = step & 1 alternates between two sets of slots: a rank can run at
// most one step ahead of the slowest one (it needs everyone's contribution to finish a step), so
// two sets are enough to keep a fast rank from overwriting what a slow one still has to read.
// All ranks must make the same sequence of calls with the same shapes.  A rank that never shows up
// makes the others' polls run out, which sets the status word and ends the kernel - nothing spins
// forever.
//
// Peer memory is touched with plain ld/st instructions only (no bulk copies, no switch reductions).
#pragma once

#include "mk36_common.cuh"

namespace mk36 {

constexpr int kCommMaxRanks = MK36_MAX_RANKS;
constexpr int kCommMaxElems = 8 * 8192;        // values per (parity, source rank): 8 tokens x hidden <= 8192
constexpr size_t kCommHeaderBytes = 4096;      // step counter
constexpr size_t kCommSlotBytes = (size_t)2 * kCommMaxRanks * kCommMaxElems * 8;
constexpr size_t kCommBytes = kCommHeaderBytes + kCommSlotBytes;
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

__device__ __forceinline__ unsigned long long* comm_slot(unsigned char* base, int parity, int src) {
    return reinterpret_cast<unsigned long long*>(base + kCommHeaderBytes) + (size_t)(parity * kCommMaxRanks + src) * kCommMaxElems;
}

__device__ __forceinline__ unsigned comm_read_step(const CommParams& c) {
    unsigned v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(comm_step_ptr(comm_buf(c, c.rank))) : "memory");
    return v;
}

__device__ __forceinline__ void comm_write_step(const CommParams& c, unsigned v) {
    asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(comm_step_ptr(comm_buf(c, c.rank))), "r"(v) : "memory");
}

// Sends element `idx` of this rank's partial sum for step `step` to every rank.
__device__ __forceinline__ void comm_put(const CommParams& c, unsigned step, size_t idx, float v) {
    const unsigned long long word = ((unsigned long long)(step + 1u) << 32) | (unsigned long long)__float_as_uint(v);
    const int parity = (int)(step & 1u);
    for (int q = 0; q < c.world; ++q) {
        asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(comm_slot(comm_buf(c, q), parity, c.rank) + idx), "l"(word) : "memory");
    }
}

// Out of line and fed with plain values: a reference to the kernel parameters would force a copy of
// the parameter block into local memory.  Returns false when the word never shows up.
static __device__ __noinline__ bool comm_poll_slow(const unsigned long long* addr, unsigned tag, Control* ctl, unsigned long long* word) {
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    for (;;) {
        unsigned long long w;
        asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w) : "l"(addr) : "memory");
        if ((unsigned)(w >> 32) == tag) {
            *word = w;
            return true;
        }
        if ((++spins & 63u) == 0u && global_timer_ns() - t0 > kCommWaitLimitNs) {
            atomicCAS(&ctl->status, 0, kStatusCommWait);
            return false;
        }
    }
}

// Sum over the ranks, in rank order, of element `idx` for step `step`; waits (bounded) for
// contributions that have not arrived yet.  Returns false when one never arrives.  The words of four ranks
// are requested before the first of them is looked at: eight dependent round trips to L2 would cost more
// than the exchange itself.
__device__ __forceinline__ bool comm_get_sum(const CommParams& c, Control* ctl, unsigned step, size_t idx, float* sum) {
    const int parity = (int)(step & 1u);
    unsigned char* own = comm_buf(c, c.rank);
    float v = 0.0f;
    // four ranks at a time: all of a batch's words in flight together without holding sixteen registers
#pragma unroll
    for (int q0 = 0; q0 < kCommMaxRanks; q0 += 4) {
        if (q0 >= c.world) break;
        unsigned long long w[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            w[j] = 0ull;
            if (q0 + j < c.world) {
                const unsigned long long* addr = comm_slot(own, parity, q0 + j) + idx;
                asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(w[j]) : "l"(addr) : "memory");
            }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (q0 + j < c.world) {
                if ((unsigned)(w[j] >> 32) != step + 1u) {
                    // once any wait of this kernel has given up the others do not start theirs: the kernel ends
                    // within one wait limit, not one per element
                    if (ld_volatile_s32(&ctl->status) != 0) return false;
                    unsigned long long late;  // not &w[j]: taking its address would move the array to local memory
                    if (!comm_poll_slow(comm_slot(own, parity, q0 + j) + idx, step + 1u, ctl, &late)) return false;
                    w[j] = late;
                }
                v += __uint_as_float((unsigned)w[j]);
            }
        }
    }
    *sum = v;
    return true;
}

#endif  // __CUDACC__

}  // namespace mk36
