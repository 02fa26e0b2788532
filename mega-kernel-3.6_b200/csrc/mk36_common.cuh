// Shared host/device helpers for the sm_100a decode kernels: error reporting, the workspace
// control block, a bounded grid-wide barrier, 128-bit streaming loads and element unpacking.
//
// Native counterpart of the reference's csrc/common.cuh (MK_CHECK_* macros, mk_silu,
// mk_warp_sum, mk_block_sum); nothing here depends on ATen.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "mk36.h"

namespace mk36 {

// ------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------
void set_error(const char* fmt, ...);

#define MK36_FAIL(code, ...)          \
    do {                              \
        ::mk36::set_error(__VA_ARGS__); \
        return (code);                \
    } while (0)

#define MK36_CUDA_OK(expr)                                                              \
    do {                                                                                \
        cudaError_t mk36_e_ = (expr);                                                   \
        if (mk36_e_ != cudaSuccess) {                                                   \
            ::mk36::set_error("%s failed: %s", #expr, cudaGetErrorString(mk36_e_));     \
            return MK36_ERR_LAUNCH;                                                     \
        }                                                                               \
    } while (0)

struct DeviceInfo {
    int device = -1;
    int sm_count = 0;
    int max_smem_optin = 0;
    int cooperative = 0;
};
// Cached per device; returns nullptr (and sets the error) when the query fails.
const DeviceInfo* current_device_info();

// Launches `kernel` so that all `grid` CTAs are co-resident (cooperative launch), which the
// grid barrier below relies on.
int launch_cooperative(const void* kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       void** params, const char* what);

// Makes sure `kernel` may be launched with `bytes` of dynamic shared memory (driver call made once
// per device, kernel and size, not per launch).
int ensure_dynamic_smem(const void* kernel, size_t bytes);

// Number of CTAs of `kernel` that fit on one SM (cached by the callers).
int max_ctas_per_sm(const void* kernel, int threads, size_t smem);

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Division by a divisor fixed at launch time: n / d == (n * mul) >> shift for every n < 2^31.
// (An integer division by a run-time value costs tens of dependent instructions on the GPU; the
// decode kernels run each code path about once, so such chains are directly visible in their time.)
struct FastDiv {
    unsigned d, mul, shift;
};
inline FastDiv make_fastdiv(unsigned d) {
    if (d == 0) d = 1;
    unsigned s = 0;
    while ((1ull << s) < d) ++s;
    FastDiv f;
    f.d = d;
    f.mul = (unsigned)(((1ull << (31 + s)) + d - 1) / d);
    f.shift = 31 + s;
    return f;
}

// Process-wide switches set through mk36_set_option (tests use them to reach every code path).
struct Options {
    int force_generic = 0;  // 1: always use the register-streaming kernels, never the ring variants
    int ring_mma = 0;       // 1: the MoE ring kernel contracts with mma.sync whatever the token count
    int moe_stream = 1;     // most tokens a call may have to run the stream kernel (0: never, 2: also two-token calls)
    int moe_batch = 1;      // 0: calls the stream kernel does not take use the ring kernel instead of the batch kernel
    int moe_stages = 0;     // > 0: ring depth of the MoE stream kernel (default: chosen from the shapes)
    int attn_stream = 1;    // 0: attention calls skip the streaming kernel (shared-memory ring) and use the register-staged one
    int dense_stream = 1;   // 0: one-token dense FFN calls use the tensor-core kernel instead of the streaming kernel
    int moe_dyn_rounds = 0; // > 0: rounds of gate/up chunks at the end of the stream dealt through the work counter (default: 4 in the stream kernel, 2 in the batch kernel)
    int linear_mma = 3;     // fewest tokens for which a projection runs on tensor-core tiles (0: never)
    int moe_static = 0;     // 1: the MoE stream kernel deals its gate/up chunks statically (no work counter)
    int static_scratch_limit = 0;  // > 0: mk36_full_attention_decode_static treats its array as this many bytes (test hook)
};
Options& options();

// ------------------------------------------------------------------------------------------
// Workspace control block (first kControlBytes of every workspace)
// ------------------------------------------------------------------------------------------
constexpr int kTraceSlots = 24;

struct Control {
    unsigned int bar_count;   // barrier arrivals since the kernel started
    unsigned int work_ticket; // next unit of dynamically dealt work (MoE stream kernel); zero between kernels
    int status;               // 0 or the code of the wait that gave up; sticky until the workspace is initialised again
    unsigned int ticket;      // CTAs that have left the kernel (see barrier_finish)
    unsigned int epoch;       // kernels that have finished on this workspace; tags the words of the mailboxes
    unsigned int reserved[11];
    // %globaltimer stamps (ns) written by CTA 0 of the last kernel that used this workspace, one
    // per phase boundary; read back with mk36_workspace_trace
    unsigned long long trace[kTraceSlots];
    // grid-wide arg-max of the projection kernel: {ordered value, ~row} per token; zero between kernels
    unsigned long long best[8];
};
// The control block is followed, inside the first kControlBytes, by per-CTA stamps: thread 0 of
// CTA c writes slot s at kCtaTraceOffset + (c * kCtaTraceSlots + s) * 8 (read back with
// mk36_workspace_cta_trace; used to see how far apart the CTAs reach a phase boundary).
constexpr size_t kCtaTraceOffset = 4096;
constexpr int kCtaTraceSlots = 8;
constexpr int kCtaTraceMaxCtas = 192;
// Mailboxes: 64-bit words {value, tag} that carry small results from every CTA to every CTA without a
// barrier.  Every receiving CTA has its own copy (kTagSlots words), so no line is polled by more than one
// CTA.  A word is valid for the running kernel when its tag is Control::epoch + 1; the epoch grows by one
// per finished kernel, so the words never need clearing.  The mailboxes sit at a fixed offset of the
// workspace that no kernel uses as scratch and mk36_workspace_init zeroes, so a stale bit pattern can
// never pass for a tag.  (MoE stream and batch kernels: router logits, [token][expert].)
constexpr int kTagSlots = 2048;
constexpr int kMailboxMaxCtas = 256;
constexpr size_t kMailboxOffset = size_t(16) << 20;
constexpr size_t kMailboxBytes = (size_t)kMailboxMaxCtas * kTagSlots * 8;
constexpr size_t kTaggedEnd = kMailboxOffset + kMailboxBytes;
constexpr size_t kControlBytes = 32768;
static_assert(sizeof(Control) <= kCtaTraceOffset, "control block too large");
static_assert(kCtaTraceOffset + (size_t)kCtaTraceMaxCtas * kCtaTraceSlots * 8 <= kControlBytes, "per-CTA trace does not fit");

// Codes stored in Control::status
constexpr int kStatusMoeBarrier1 = 101;
constexpr int kStatusMoeBarrier2 = 102;
constexpr int kStatusMoeRingProducer = 111;  // producer warp: a stage was never released
constexpr int kStatusMoeRingConsumer = 112;  // consumer warp: a stage never filled
constexpr int kStatusLinearProducer = 131;   // projection kernel: a stage was never released
constexpr int kStatusLinearConsumer = 132;   // projection kernel: a stage never filled
constexpr int kStatusMoeLogits = 121;        // stream kernel: another CTA's router logits never arrived
constexpr int kStatusDenseBarrier = 201;
constexpr int kStatusAttnBarrier = 301;
constexpr int kStatusSelfTest = 901;

// Bounded waits give up after this long (nanoseconds of %globaltimer).
constexpr unsigned long long kWaitLimitNs = 400ull * 1000ull * 1000ull;

#if defined(__CUDACC__)
// ------------------------------------------------------------------------------------------
// Device side
// ------------------------------------------------------------------------------------------
constexpr unsigned kFullMask = 0xffffffffu;

__device__ __forceinline__ int fdiv(int n, const FastDiv& f) {
    return (int)(((unsigned long long)(unsigned)n * f.mul) >> f.shift);
}
__device__ __forceinline__ void fdivmod(int n, const FastDiv& f, int& q, int& r) {
    q = fdiv(n, f);
    r = n - q * (int)f.d;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Phase stamp for the workspace trace; call from one thread of CTA 0.
__device__ __forceinline__ void trace_stamp(Control* c, int slot) {
    if (slot < kTraceSlots) c->trace[slot] = global_timer_ns();
}

// Per-CTA stamp; call from one thread of each CTA.
__device__ __forceinline__ void cta_stamp(Control* c, int cta, int slot) {
    if (cta < kCtaTraceMaxCtas && slot < kCtaTraceSlots) {
        unsigned long long* base = reinterpret_cast<unsigned long long*>(reinterpret_cast<unsigned char*>(c) + kCtaTraceOffset);
        base[cta * kCtaTraceSlots + slot] = global_timer_ns();
    }
}

__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Grid barrier on a counter that only grows during a launch.  Barrier number `ordinal` (0, 1, ...
// in the order the kernel reaches them) is complete when the counter has reached
// (ordinal + 1) * nblocks, so the last arrival is visible to the waiters with one atomic and one
// poll; the counter is put back to zero by the last CTA that leaves the kernel (barrier_finish),
// which is safe because kernels that share a workspace are ordered by their stream.
// All CTAs of a co-resident grid call arrive() then wait() for every ordinal, and barrier_finish()
// once at the end.  arrive() must be preceded by a CTA-wide sync issued by the caller when the CTA's
// earlier global writes have to be visible to the other CTAs after their wait().
// Only one thread of a CTA touches the counters.  Returns the target for the matching wait.
__device__ __forceinline__ unsigned barrier_arrive(Control* c, unsigned nblocks, unsigned ordinal = 0) {
    asm volatile("red.release.gpu.global.add.u32 [%0], 1;" ::"l"(&c->bar_count) : "memory");
    return (ordinal + 1u) * nblocks;
}

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ int ld_volatile_s32(const int* p) {
    int v;
    asm volatile("ld.volatile.global.s32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Returns false when the wait ran out; the status word then holds `code`.  A status word that is
// already set makes every wait fail at once: after a wait has given up the counters are left dirty
// (the CTAs that gave up never reach barrier_finish), so nothing may compute on this workspace
// until the host has initialised it again, and the kernels queued behind the failure leave their
// outputs untouched.
__device__ __forceinline__ bool barrier_wait(Control* c, unsigned target, int code,
                                             unsigned long long limit_ns = kWaitLimitNs) {
    const int dirty = ld_volatile_s32(&c->status);  // issued before the acquire load: both are in flight together
    const unsigned seen = ld_acquire_u32(&c->bar_count);
    if (dirty != 0) return false;
    if (seen >= target) return true;
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (ld_acquire_u32(&c->bar_count) < target) {
        if ((++spins & 63u) == 0u) {
            if (global_timer_ns() - t0 > limit_ns) {
                atomicCAS(&c->status, 0, code);
                return false;
            }
        }
    }
    return true;
}

// Called by one thread of every CTA after its last barrier wait: the last CTA to leave resets the
// counters for the next kernel on this workspace.  CTAs that gave up on a wait do not call it (the
// workspace then has to be initialised again).
__device__ __forceinline__ void barrier_finish(Control* c, unsigned nblocks) {
    if (atomicAdd(&c->ticket, 1u) == nblocks - 1u) {
        c->bar_count = 0u;
        c->work_ticket = 0u;
        c->ticket = 0u;
        c->epoch = c->epoch + 1u;
        __threadfence();
    }
}

// Full barrier for a whole CTA (every thread calls it).  Returns a CTA-uniform flag.
__device__ __forceinline__ bool grid_barrier(Control* c, unsigned nblocks, unsigned ordinal, int code, int* s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned target = barrier_arrive(c, nblocks, ordinal);
        *s_flag = barrier_wait(c, target, code) ? 1 : 0;
    }
    __syncthreads();
    return *s_flag != 0;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(kFullMask, v, off);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) v = fmaxf(v, __shfl_xor_sync(kFullMask, v, off));
    return v;
}

// silu(x) = x / (1 + exp(-x)) with the accurate expf (no fast-math), as torch's fp32 silu.
__device__ __forceinline__ float silu(float v) { return v / (1.0f + expf(-v)); }

// ---- element conversion --------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float to_float(T v);
template <>
__device__ __forceinline__ float to_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <>
__device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }

template <typename T>
__device__ __forceinline__ T from_float(float v);
template <>
__device__ __forceinline__ float from_float<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <>
__device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }

// Round to the storage type and widen again (the reference rounds the normalised input to the
// activation dtype before the projections).
template <typename T>
__device__ __forceinline__ float round_through(float v) { return to_float<T>(from_float<T>(v)); }

// ---- streaming loads of 8 consecutive elements ---------------------------------------------
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

template <typename T>
struct Chunk8 {  // 2-byte element types: 16 bytes
    uint4 raw;
};
template <>
struct Chunk8<float> {
    uint4 lo, hi;
};

template <typename T>
__device__ __forceinline__ Chunk8<T> load_chunk8(const T* p) {
    Chunk8<T> c;
    c.raw = ld_stream_u4(p);
    return c;
}
template <>
__device__ __forceinline__ Chunk8<float> load_chunk8<float>(const float* p) {
    Chunk8<float> c;
    c.lo = ld_stream_u4(p);
    c.hi = ld_stream_u4(p + 4);
    return c;
}

template <typename T>
__device__ __forceinline__ void zero_chunk8(Chunk8<T>& c) { c.raw = make_uint4(0, 0, 0, 0); }
template <>
__device__ __forceinline__ void zero_chunk8<float>(Chunk8<float>& c) {
    c.lo = make_uint4(0, 0, 0, 0);
    c.hi = make_uint4(0, 0, 0, 0);
}

__device__ __forceinline__ void unpack8(const Chunk8<__nv_bfloat16>& c, float (&f)[8]) {
    // a bf16 is the upper half of an fp32
    f[0] = __uint_as_float(c.raw.x << 16);
    f[1] = __uint_as_float(c.raw.x & 0xffff0000u);
    f[2] = __uint_as_float(c.raw.y << 16);
    f[3] = __uint_as_float(c.raw.y & 0xffff0000u);
    f[4] = __uint_as_float(c.raw.z << 16);
    f[5] = __uint_as_float(c.raw.z & 0xffff0000u);
    f[6] = __uint_as_float(c.raw.w << 16);
    f[7] = __uint_as_float(c.raw.w & 0xffff0000u);
}
__device__ __forceinline__ void unpack8(const Chunk8<__half>& c, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&c.raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        float2 t = __half22float2(h[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}
__device__ __forceinline__ void unpack8(const Chunk8<float>& c, float (&f)[8]) {
    f[0] = __uint_as_float(c.lo.x);
    f[1] = __uint_as_float(c.lo.y);
    f[2] = __uint_as_float(c.lo.z);
    f[3] = __uint_as_float(c.lo.w);
    f[4] = __uint_as_float(c.hi.x);
    f[5] = __uint_as_float(c.hi.y);
    f[6] = __uint_as_float(c.hi.z);
    f[7] = __uint_as_float(c.hi.w);
}

// Activation vectors live in shared memory as fp32 in a split layout: element k of a vector of
// (padded) length 8*nchunks sits at  (k/8)*4 + (k%4)  in the first half when (k%8) < 4 and at the
// same offset in the second half otherwise, so that a warp reading chunk `lane` issues two
// conflict-free 128-bit loads.
__device__ __forceinline__ int split_index(int k, int half_floats) {
    return ((k >> 3) << 2) + (k & 3) + ((k & 4) ? half_floats : 0);
}

#endif  // __CUDACC__

}  // namespace mk36
