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

// Number of CTAs of `kernel` that fit on one SM (cached by the callers).
int max_ctas_per_sm(const void* kernel, int threads, size_t smem);

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Process-wide switches set through mk36_set_option (tests use them to reach every code path).
struct Options {
    int force_generic = 0;  // 1: always use the register-streaming kernels, never the ring variants
};
Options& options();

// ------------------------------------------------------------------------------------------
// Workspace control block (first kControlBytes of every workspace)
// ------------------------------------------------------------------------------------------
constexpr int kTraceSlots = 16;

struct Control {
    unsigned int bar_count;   // arrivals at the current barrier
    unsigned int bar_gen;     // completed barriers (monotone)
    int status;               // 0 or the code of the wait that gave up
    unsigned int ticket;      // general purpose arrival ticket
    unsigned int reserved[12];
    // %globaltimer stamps (ns) written by CTA 0 of the last kernel that used this workspace, one
    // per phase boundary; read back with mk36_workspace_trace
    unsigned long long trace[kTraceSlots];
};
constexpr size_t kControlBytes = 4096;
static_assert(sizeof(Control) <= kControlBytes, "control block too large");

// Codes stored in Control::status
constexpr int kStatusMoeBarrier1 = 101;
constexpr int kStatusMoeBarrier2 = 102;
constexpr int kStatusMoeRingProducer = 111;  // producer warp: a stage was never released
constexpr int kStatusMoeRingConsumer = 112;  // consumer warp: a stage never filled
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

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Phase stamp for the workspace trace; call from one thread of CTA 0.
__device__ __forceinline__ void trace_stamp(Control* c, int slot) {
    if (slot < kTraceSlots) c->trace[slot] = global_timer_ns();
}

__device__ __forceinline__ unsigned ld_volatile_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

// Split grid barrier.  All CTAs of a co-resident grid call arrive() then wait() the same number
// of times.  arrive() must be preceded by a __syncthreads() issued by the caller when the CTA's
// earlier global writes have to be visible to the other CTAs after their wait().
// Only thread 0 of a CTA touches the counters.
__device__ __forceinline__ unsigned barrier_arrive(Control* c, unsigned nblocks) {
    unsigned gen = ld_volatile_u32(&c->bar_gen);
    __threadfence();
    unsigned prev = atomicAdd(&c->bar_count, 1u);
    if (prev == nblocks - 1) {
        atomicExch(&c->bar_count, 0u);
        __threadfence();
        atomicAdd(&c->bar_gen, 1u);
    }
    return gen;
}

// Returns false when the wait ran out; the status word then holds `code`.
__device__ __forceinline__ bool barrier_wait(Control* c, unsigned gen, int code,
                                             unsigned long long limit_ns = kWaitLimitNs) {
    if (ld_volatile_u32(&c->bar_gen) != gen) {
        __threadfence();
        return true;
    }
    const unsigned long long t0 = global_timer_ns();
    unsigned spins = 0;
    while (ld_volatile_u32(&c->bar_gen) == gen) {
        if ((++spins & 63u) == 0u) {
            if (global_timer_ns() - t0 > limit_ns) {
                atomicCAS(&c->status, 0, code);
                return false;
            }
        }
    }
    __threadfence();
    return true;
}

// Full barrier for a whole CTA (every thread calls it).  Returns a CTA-uniform flag.
__device__ __forceinline__ bool grid_barrier(Control* c, unsigned nblocks, int code, int* s_flag) {
    __syncthreads();
    if (threadIdx.x == 0) {
        unsigned gen = barrier_arrive(c, nblocks);
        *s_flag = barrier_wait(c, gen, code) ? 1 : 0;
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
