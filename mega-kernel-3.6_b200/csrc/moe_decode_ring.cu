// MoE decode, streaming variant for sm_100a (2-byte dtypes, aligned shapes).
//
// Same phases and results as the general kernel in moe_decode.cu, organised around two facts
// measured on B200: a cold HBM access costs 2-3 us, and at batch <= 8 the scalar unpack + FMA
// work per weight element is as expensive as streaming it.  So
//   * the weights do not go through registers on their way from HBM: one producer lane feeds a
//     shared-memory ring of 32 KB stages with 1-D bulk copies (cp.async.bulk completing on
//     mbarriers, each copy into the issuing CTA only).  Weight addresses depend only on the routing decision, so the
//     producer runs ahead of the grid barriers: router rows, shared-expert rows and the CTA's
//     slice of shared_down are requested at kernel entry, before the token is even normalised,
//     and once the top-k is known the routed gate/up rows and then the routed down rows are
//     requested back to back, so the down rows are in shared memory (or in flight) while the
//     second grid barrier completes;
//   * the twelve consumer warps contract with the warp-level tensor-core instruction
//     mma.sync.m16n8k16 (bf16/f16 in, fp32 accumulate): weight rows are the M side (16 rows), the
//     tokens of the launch are the N side (8 columns), so all tokens are served by the same
//     instruction stream and one weight byte costs ~1/8 of the instructions of the scalar path.
//     The normalised token is exactly representable in the activation dtype (the reference rounds
//     it), so it is an exact MMA operand; fp32 activations of the down projection are split into a
//     high and a low half (two MMAs) and lose nothing.
//
//   stream of one CTA:  [router rows][shared gate+up rows] | [routed gate+up rows][routed down rows]
//                        issued at entry                      issued after the top-k
//
// A stage holds up to `rows_h` router rows, or gate rows i..i+n and (second half) up rows i..i+n
// of one expert so that silu(gate_i.x) * (up_i.x) is formed without a trip through memory, or this
// CTA's output rows of the down projection of up to `epc` experts.  Stage n is consumed by warp
// group n % 3.  Partial results per (token, slot) pair are kept apart and summed in slot order at the
// end, so the result does not depend on timing.
#include <cfloat>
#include <climits>

#include "mk36_comm.cuh"
#include "mk36_mma.cuh"
#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kRingConsumerWarps = 12;  // 12 + 1 producer: 13 warps are allocated as 16, i.e. 128 registers per thread
constexpr int kRingConsumerThreads = kRingConsumerWarps * 32;
constexpr int kRingThreads = kRingConsumerThreads + 32;  // + one producer warp
constexpr int kRingStageBytes = 32768;  // bulk copies under 16 KB cost bandwidth; 32 KB x 3..6 stages streams at the HBM rate
constexpr int kRingGroups = 3;
constexpr int kRingGroupWarps = kRingConsumerWarps / kRingGroups;
constexpr int kRingGroupThreads = kRingGroupWarps * 32;
constexpr int kRingMaxStages = 6;   // kRingGroups x (1 or 2)
constexpr int kRingMaxDed = 4;      // single-use slots for the first down-projection chunks
constexpr int kRingMaxTokens = 8;   // = N of the MMA tile
constexpr int kRingMaxPairs = 64;
constexpr int kRingTileRows = 16;   // = M of the MMA tile
constexpr int kTopkPerLane = 8;     // register top-k: experts <= 256
constexpr int kActBatch = 4;        // 16-byte activation loads in flight per thread

struct MoeRingParams {
    const void* x;
    const void* norm_w;
    const void* router_w;
    const void* egate;
    const void* eup;
    const void* edown;
    const void* sgate;
    const void* sup;
    const void* sdown;
    void* out;
    long long* indices;
    float* route_w;
    float* partial_out;
    Control* ctl;
    float* logits;  // [ntok][E]
    float* act;     // [ntok*K][I]   silu(gate) * up of the routed pairs
    float* sact;    // [ntok][Is]    same for the shared expert
    int ntok, H, E, K, I, Is;
    int expert_base, local_experts, add_residual;
    float eps;
    int nstages;
    int nded;     // shared memory left over by the ring, in stage-sized single-use slots (see off_ded)
    int rows_h;   // rows of length H per stage (<= 16, even; pairs per stage = rows_h / 2)
    int epc;      // experts per stage in the down phase (<= 4)
    int hr_max;   // max output rows per CTA (<= 16)
    int scalar;   // 1: at most two tokens in the launch, contract with plain FMAs instead of mma.sync
    int log2_depth;   // stages per consumer group = 1 << log2_depth; nstages = kRingGroups << log2_depth
    FastDiv fd_ncta, fd_rows_h, fd_pr, fd_I, fd_K, fd_qi, fd_qis, fd_epc, fd_ks;
    // byte offsets into dynamic shared memory
    int off_ded, off_ring, off_sdown, off_act, off_part, off_red, off_logits, off_uniq_e, off_uniq_m, off_pair_e, off_pair_w, off_bars;
    CommParams comm;  // world > 1: the epilogue sums the ranks' partial outputs over peer memory
};

__device__ __forceinline__ int chunks_in(int r0, int r1, const FastDiv& per) {
    return r1 > r0 ? (fdiv(r1 - 1, per) - fdiv(r0, per) + 1) : 0;
}

// items [first, first + count) of chunk n of the range [r0, r1), chunks aligned to multiples of `per`;
// m0 = r0 / per is computed once by the caller
__device__ __forceinline__ void chunk_span(int r0, int r1, int per, int m0, int n, int& first, int& count) {
    const int m = m0 + n;
    const int a = max(m * per, r0);
    const int b = min((m + 1) * per, r1);
    first = a;
    count = b - a;
}

template <typename T>
__device__ __forceinline__ void unpack_u4(const uint4& v, float (&f)[8]) {
    Chunk8<T> c;
    c.raw = v;
    unpack8(c, f);
}

__device__ __forceinline__ void add4(float (&d)[4], const float (&s)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] += s[i];
}

// Tile of `nrows` (<= 16) rows of length `len` (multiple of 32) in shared memory, row r at
// base + r * row_stride elements, against up to 8 vectors of T in shared memory, vector c at
// vecs + c * vec_stride (c < ncols).  The warp takes the 32-wide slices kb = 32 * (first + step * i).
// mma.sync has a latency of tens of cycles on this part, so the sum is spread over four
// independent accumulators (two slices in flight, two MMAs per slice) and folded at the end.
template <typename T>
__device__ __noinline__ void tile_times_vectors(float (&d)[4], const T* base, int row_stride, int nrows, const T* vecs,
                                                   int vec_stride, int ncols, int len, int first, int step, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const bool row_lo = g < nrows, row_hi = (g + 8) < nrows, col = g < ncols;
    const T* a_lo = base + (size_t)g * row_stride + 8 * t;
    const T* a_hi = base + (size_t)(g + 8) * row_stride + 8 * t;
    const T* b = vecs + (size_t)g * vec_stride + 8 * t;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    float e0[4] = {0.f, 0.f, 0.f, 0.f}, e1[4] = {0.f, 0.f, 0.f, 0.f}, e2[4] = {0.f, 0.f, 0.f, 0.f}, e3[4] = {0.f, 0.f, 0.f, 0.f};
    int kb = 32 * first;
    for (; kb + 32 * step < len; kb += 64 * step) {
        const int kc = kb + 32 * step;
        const uint4 va = row_lo ? lds128(a_lo + kb) : zero;
        const uint4 vb = row_hi ? lds128(a_hi + kb) : zero;
        const uint4 vx = col ? lds128(b + kb) : zero;
        const uint4 wa = row_lo ? lds128(a_lo + kc) : zero;
        const uint4 wb = row_hi ? lds128(a_hi + kc) : zero;
        const uint4 wx = col ? lds128(b + kc) : zero;
        mma_slice32<T>(e0, e1, va, vb, vx);
        mma_slice32<T>(e2, e3, wa, wb, wx);
    }
    if (kb < len) {
        const uint4 va = row_lo ? lds128(a_lo + kb) : zero;
        const uint4 vb = row_hi ? lds128(a_hi + kb) : zero;
        const uint4 vx = col ? lds128(b + kb) : zero;
        mma_slice32<T>(e0, e1, va, vb, vx);
    }
    add4(e0, e1);
    add4(e2, e3);
    add4(e0, e2);
    add4(d, e0);
}

// Same with two sets of vectors (high and low halves of fp32 activations) sharing the tile loads.
// `col_hi` / `col_lo` point at this lane's column (column index = lane / 4) or are null when the
// column is unused; the whole length is contracted by this warp.  Eight independent accumulators.
template <typename T>
__device__ __noinline__ void tile_times_split_vectors(float (&d)[4], const T* base, int row_stride, int nrows,
                                                         const T* col_hi, const T* col_lo, int len, int lane) {
    const int g = lane >> 2, t = lane & 3;
    const bool row_lo = g < nrows, row_hi = (g + 8) < nrows, col = col_hi != nullptr;
    const T* a_lo = base + (size_t)g * row_stride + 8 * t;
    const T* a_hi = base + (size_t)(g + 8) * row_stride + 8 * t;
    const T* bh = col_hi + 8 * t;
    const T* bl = col_lo + 8 * t;
    const uint4 zero = make_uint4(0, 0, 0, 0);
    float e[8][4];
#pragma unroll
    for (int i = 0; i < 8; ++i) { e[i][0] = 0.f; e[i][1] = 0.f; e[i][2] = 0.f; e[i][3] = 0.f; }
    int kb = 0;
    for (; kb + 32 < len; kb += 64) {
        const uint4 va = row_lo ? lds128(a_lo + kb) : zero;
        const uint4 vb = row_hi ? lds128(a_hi + kb) : zero;
        const uint4 xh = col ? lds128(bh + kb) : zero;
        const uint4 xl = col ? lds128(bl + kb) : zero;
        const uint4 wa = row_lo ? lds128(a_lo + kb + 32) : zero;
        const uint4 wb = row_hi ? lds128(a_hi + kb + 32) : zero;
        const uint4 yh = col ? lds128(bh + kb + 32) : zero;
        const uint4 yl = col ? lds128(bl + kb + 32) : zero;
        mma_slice32<T>(e[0], e[1], va, vb, xh);
        mma_slice32<T>(e[2], e[3], va, vb, xl);
        mma_slice32<T>(e[4], e[5], wa, wb, yh);
        mma_slice32<T>(e[6], e[7], wa, wb, yl);
    }
    if (kb < len) {
        const uint4 va = row_lo ? lds128(a_lo + kb) : zero;
        const uint4 vb = row_hi ? lds128(a_hi + kb) : zero;
        const uint4 xh = col ? lds128(bh + kb) : zero;
        const uint4 xl = col ? lds128(bl + kb) : zero;
        mma_slice32<T>(e[0], e[1], va, vb, xh);
        mma_slice32<T>(e[2], e[3], va, vb, xl);
    }
    add4(e[0], e[1]); add4(e[2], e[3]); add4(e[4], e[5]); add4(e[6], e[7]);
    add4(e[0], e[2]); add4(e[4], e[6]);
    add4(e[0], e[4]);
    add4(d, e[0]);
}

// ---- plain-FMA contraction for launches of one or two tokens ----
// On this part a warp-level mma.sync costs tens of issue cycles, so for a handful of token columns
// unpack + FMA needs several times fewer cycles than the tensor-core instruction that computes
// eight columns at once.  A warp takes whole rows (no partial tiles to combine, hence no barrier
// between the warps of a group): lane l reads the 16-byte pieces l, l + 32, ... of the row, which
// is conflict-free in shared memory, and the warp reduces with shuffles.

// Dot products of row `ra` (and, when PAIR, row `rb`) of `nchunks` 8-element pieces with NT vectors of T.
template <typename T, int NT, bool PAIR>
__device__ __forceinline__ void dot_rows_t(const T* ra, const T* rb, const T* const (&xp)[NT], int nchunks, int lane, float (&sa)[NT],
                                           float (&sb)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) { sa[t] = 0.0f; sb[t] = 0.0f; }
#pragma unroll 2
    for (int c = lane; c < nchunks; c += 32) {
        float fa[8], fb[8];
        unpack_u4<T>(lds128(ra + 8 * c), fa);
        if (PAIR) unpack_u4<T>(lds128(rb + 8 * c), fb);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float fx[8];
            unpack_u4<T>(lds128(xp[t] + 8 * c), fx);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sa[t] = fmaf(fa[i], fx[i], sa[t]);
                if (PAIR) sb[t] = fmaf(fb[i], fx[i], sb[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        sa[t] = warp_sum(sa[t]);
        if (PAIR) sb[t] = warp_sum(sb[t]);
    }
}

// One (gate, up) pair or one single row against one or two token vectors; results in ga[j] / ua[j]
// (ua only when rb is given).
template <typename T>
__device__ __forceinline__ void rows_times_tokens(const T* ra, const T* rb, const T* x0, const T* x1, const T* x2, const T* x3, int nvec,
                                               int nchunks, int lane, float (&ga)[4], float (&ua)[4]) {
    if (nvec <= 1) {
        const T* const xp[1] = {x0};
        float a[1], b[1];
        if (rb) dot_rows_t<T, 1, true>(ra, rb, xp, nchunks, lane, a, b);
        else dot_rows_t<T, 1, false>(ra, rb, xp, nchunks, lane, a, b);
        ga[0] = a[0]; ua[0] = b[0];
    } else {  // the plain-FMA path is only taken for launches of one or two tokens
        const T* const xp[2] = {x0, x1};
        float a[2], b[2];
        if (rb) dot_rows_t<T, 2, true>(ra, rb, xp, nchunks, lane, a, b);
        else dot_rows_t<T, 2, false>(ra, rb, xp, nchunks, lane, a, b);
        ga[0] = a[0]; ga[1] = a[1]; ua[0] = b[0]; ua[1] = b[1];
    }
}

// Down projection, plain-FMA path: four lanes share a row (lane t of the four takes the 16-byte pieces
// t, t + 4, ...), so a warp works on eight rows at once and one pass of a group's four warps covers a
// whole chunk; many independent rows in flight instead of one latency chain per row.  The
// activations are fp32 in shared memory; lanes on different rows read the same activation
// address (a broadcast).  Returns the quad-reduced sums in every lane of the quad.
template <typename T, int NT>
__device__ __forceinline__ void quad_row_dot(const T* row, const float* const (&ap)[NT], int nchunks, int t4, float (&s)[NT]) {
    float s2[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) { s[t] = 0.0f; s2[t] = 0.0f; }
    int c = t4;
    for (; c + 4 < nchunks; c += 8) {
        float f[8], g[8];
        unpack_u4<T>(lds128(row + 8 * c), f);
        unpack_u4<T>(lds128(row + 8 * (c + 4)), g);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float4 a = *reinterpret_cast<const float4*>(ap[t] + 8 * c);
            const float4 b = *reinterpret_cast<const float4*>(ap[t] + 8 * c + 4);
            const float4 a2 = *reinterpret_cast<const float4*>(ap[t] + 8 * (c + 4));
            const float4 b2 = *reinterpret_cast<const float4*>(ap[t] + 8 * (c + 4) + 4);
            float v = s[t], w = s2[t];
            v = fmaf(f[0], a.x, v); w = fmaf(g[0], a2.x, w);
            v = fmaf(f[1], a.y, v); w = fmaf(g[1], a2.y, w);
            v = fmaf(f[2], a.z, v); w = fmaf(g[2], a2.z, w);
            v = fmaf(f[3], a.w, v); w = fmaf(g[3], a2.w, w);
            v = fmaf(f[4], b.x, v); w = fmaf(g[4], b2.x, w);
            v = fmaf(f[5], b.y, v); w = fmaf(g[5], b2.y, w);
            v = fmaf(f[6], b.z, v); w = fmaf(g[6], b2.z, w);
            v = fmaf(f[7], b.w, v); w = fmaf(g[7], b2.w, w);
            s[t] = v; s2[t] = w;
        }
    }
    for (; c < nchunks; c += 4) {
        float f[8];
        unpack_u4<T>(lds128(row + 8 * c), f);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            const float4 a = *reinterpret_cast<const float4*>(ap[t] + 8 * c);
            const float4 b = *reinterpret_cast<const float4*>(ap[t] + 8 * c + 4);
            float v = s[t];
            v = fmaf(f[0], a.x, v); v = fmaf(f[1], a.y, v); v = fmaf(f[2], a.z, v); v = fmaf(f[3], a.w, v);
            v = fmaf(f[4], b.x, v); v = fmaf(f[5], b.y, v); v = fmaf(f[6], b.z, v); v = fmaf(f[7], b.w, v);
            s[t] = v;
        }
    }
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        float v = s[t] + s2[t];
        v += __shfl_xor_sync(kFullMask, v, 1);
        v += __shfl_xor_sync(kFullMask, v, 2);
        s[t] = v;
    }
}

// position of the q-th set bit of m (q < popcount(m))
__device__ __forceinline__ int nth_set_bit(unsigned long long m, int q) {
    for (int i = 0; i < q; ++i) m &= m - 1;
    return __ffsll((long long)m) - 1;
}

template <typename T, bool SC>
__global__ void __launch_bounds__(kRingThreads, 1) moe_decode_ring_kernel(const MoeRingParams p) {
    // SC: plain-FMA consumers (launches of one or two tokens) or tensor-core consumers.  A template
    // parameter, not a run-time flag: the kernel runs every code path about once, so the size of the
    // code it has to fetch shows in its time, and each instantiation carries only its own path.
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_unique;
    __shared__ int s_abort;
    __shared__ float s_red[kRingConsumerWarps];
    __shared__ unsigned s_step;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kRingConsumerWarps);

    unsigned char* ring = smem + p.off_ring;
    T* sdown_buf = reinterpret_cast<T*>(smem + p.off_sdown);
    T* xs = reinterpret_cast<T*>(smem + p.off_act);      // phases A/B: tokens as T [ntok][H]
    T* acts_hi = reinterpret_cast<T*>(smem + p.off_act); // phase C: activations, high halves, then low halves
    float* part = reinterpret_cast<float*>(smem + p.off_part);  // [npairs + ntok][hr_max]
    float* red = reinterpret_cast<float*>(smem + p.off_red);    // [groups][2][group warps][16][8]
    float* s_logits = reinterpret_cast<float*>(smem + p.off_logits);
    int* s_uniq_e = reinterpret_cast<int*>(smem + p.off_uniq_e);
    unsigned long long* s_uniq_m = reinterpret_cast<unsigned long long*>(smem + p.off_uniq_m);
    int* s_pair_e = reinterpret_cast<int*>(smem + p.off_pair_e);
    float* s_pair_w = reinterpret_cast<float*>(smem + p.off_pair_w);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_bar = full_bar + kRingMaxStages;
    unsigned long long* sdown_bar = empty_bar + kRingMaxStages;
    unsigned long long* ded_bar = sdown_bar + 1;
    unsigned char* ded = smem + p.off_ded;

    const T* x = static_cast<const T*>(p.x);
    const int NS = p.nstages;
    const size_t rowH = (size_t)p.H;          // elements per row of length hidden
    const int PR = p.rows_h >> 1;             // (gate, up) pairs per stage
    const size_t up_off = (size_t)PR * rowH;  // element offset of the up rows inside a stage

    // ---- static partition of this CTA's work ----
    const int r0 = fdiv(p.E * cta, p.fd_ncta), r1 = fdiv(p.E * (cta + 1), p.fd_ncta);
    const int s0 = fdiv(p.Is * cta, p.fd_ncta), s1 = fdiv(p.Is * (cta + 1), p.fd_ncta);
    const int h0 = fdiv(p.H * cta, p.fd_ncta), h1 = fdiv(p.H * (cta + 1), p.fd_ncta);
    const int hr = h1 - h0;
    const int nA1 = chunks_in(r0, r1, p.fd_rows_h);
    const int nA2 = chunks_in(s0, s1, p.fd_pr);
    const int nA = nA1 + nA2;
    const int mA1 = fdiv(r0, p.fd_rows_h), mA2 = fdiv(s0, p.fd_pr);
    // Chunk n belongs to consumer group n % 3 and lives in one of that group's own stages, so the
    // barriers of a stage are only ever waited on by one group, which walks its chunks in order and
    // therefore sees every barrier phase exactly once.  (With stages shared between groups a group
    // could look at a barrier one phase early and be told that the previous phase is complete.)
    const int depth_mask = (1 << p.log2_depth) - 1;
    auto stage_of = [&](int n) { return ((n % kRingGroups) << p.log2_depth) + ((n / kRingGroups) & depth_mask); };
    auto use_of = [&](int n) { return (n / kRingGroups) >> p.log2_depth; };  // how many times the stage was used before

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);
    if (tid == 0) cta_stamp(p.ctl, cta, 3);

    if (tid == 0) {
        s_abort = 0;
        s_step = (p.comm.world > 1) ? comm_read_step(p.comm) : 0u;
        for (int s = 0; s < kRingMaxStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kRingGroupWarps);
        }
        mbar_init(sdown_bar, 1);
        for (int s = 0; s < kRingMaxDed; ++s) mbar_init(&ded_bar[s], 1);
        mbar_init_fence();
    }
    __syncthreads();

    // =====================================================================================
    // Producer warp.  One lane issues: a bulk copy costs about a quarter of a microsecond to issue
    // however it is spread over lanes, so the number of copies, not of lanes, is what matters.
    // =====================================================================================
    if (is_producer) {
        bool ok = true;
        // chunk n goes to stage n % NS once the consumers of chunk n - NS have released it
        auto acquire = [&](int n, unsigned bytes) -> unsigned char* {
            const int stage = stage_of(n);
            if (use_of(n) > 0) ok = mbar_wait(&empty_bar[stage], (use_of(n) - 1) & 1, &s_abort);
            if (!ok) return nullptr;
            mbar_arrive_expect_tx(&full_bar[stage], bytes);
            return ring + (size_t)stage * kRingStageBytes;
        };
        if (lane == 0) {
            for (int n = 0; n < nA && ok; ++n) {
                int first, count;
                if (n < nA1) {
                    chunk_span(r0, r1, p.rows_h, mA1, n, first, count);
                    const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                    unsigned char* dst = acquire(n, bytes);
                    if (dst) bulk_copy_g2s(dst, static_cast<const T*>(p.router_w) + (size_t)first * rowH, bytes, &full_bar[stage_of(n)]);
                } else {
                    chunk_span(s0, s1, PR, mA2, n - nA1, first, count);
                    const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                    unsigned char* dst = acquire(n, 2 * bytes);
                    if (dst) {
                        bulk_copy_g2s(dst, static_cast<const T*>(p.sgate) + (size_t)first * rowH, bytes, &full_bar[stage_of(n)]);
                        bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.sup) + (size_t)first * rowH, bytes, &full_bar[stage_of(n)]);
                    }
                }
            }
            // shared_down rows of this CTA: needed only in the last phase
            if (hr > 0 && p.Is > 0) {
                const unsigned bytes = (unsigned)((size_t)hr * p.Is * sizeof(T));
                mbar_arrive_expect_tx(sdown_bar, bytes);
                bulk_copy_g2s(sdown_buf, static_cast<const T*>(p.sdown) + (size_t)h0 * p.Is, bytes, sdown_bar);
            }
        }
        __syncthreads();  // (S1) routing is known
        const int n_unique = s_unique;
        if (s_abort != 0) ok = false;
        if (lane == 0 && ok) {
            const int tasks = p.I * n_unique;
            // whole chunks per CTA (a chunk never straddles two CTAs: a partial chunk costs a full stage round trip)
    const int nch_all = fdiv(tasks, p.fd_pr);
    const int t0 = fdiv(nch_all * cta, p.fd_ncta) * PR, t1 = fdiv(nch_all * (cta + 1), p.fd_ncta) * PR;
            const int nB = chunks_in(t0, t1, p.fd_pr);
            const int mB = fdiv(t0, p.fd_pr);
            const int nC = (hr > 0) ? fdiv(n_unique + p.epc - 1, p.fd_epc) : 0;
            const int nd = min(p.nded, nC);  // down chunks that get a slot of their own
            const unsigned cbytes = (unsigned)((size_t)hr * p.I * sizeof(T));
            auto issue_down = [&](int k, unsigned char* dst, unsigned long long* bar) {
                const int ua = k * p.epc, ub = min(n_unique, ua + p.epc);
                for (int u = ua; u < ub; ++u) {
                    const int e = s_uniq_e[u] - p.expert_base;
                    bulk_copy_g2s(dst + (size_t)(u - ua) * p.hr_max * p.I * sizeof(T),
                                  static_cast<const T*>(p.edown) + ((size_t)e * p.H + h0) * p.I, cbytes, bar);
                }
            };
            auto down_bytes = [&](int k) { return cbytes * (unsigned)(min(n_unique, (k + 1) * p.epc) - k * p.epc); };
            for (int k = 0; k < nB && ok; ++k) {
                if (k == NS || (k == nB - 1 && nB <= NS)) {
                    // The ring is full of gate/up rows (or they are all requested): now ask for the down rows
                    // that have a slot of their own.  They are not needed before the second grid barrier, and
                    // requesting them here keeps them out of the way of the first gate/up rows.
                    if (cta == 0) trace_stamp(p.ctl, 17);
                    for (int c = 0; c < nd; ++c) {
                        mbar_arrive_expect_tx(&ded_bar[c], down_bytes(c));
                        issue_down(c, ded + (size_t)c * kRingStageBytes, &ded_bar[c]);
                    }
                }
                int first, count, u, i;
                chunk_span(t0, t1, PR, mB, k, first, count);
                fdivmod(first, p.fd_I, u, i);
                const int e = s_uniq_e[u] - p.expert_base;
                const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                const int n = nA + k;
                unsigned char* dst = acquire(n, 2 * bytes);
                if (cta == 0 && k == 0) trace_stamp(p.ctl, 15);
                if (cta == 0 && k == nB - 1) trace_stamp(p.ctl, 16);
                if (dst) {
                    const size_t off = ((size_t)e * p.I + i) * rowH;
                    bulk_copy_g2s(dst, static_cast<const T*>(p.egate) + off, bytes, &full_bar[stage_of(n)]);
                    bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.eup) + off, bytes, &full_bar[stage_of(n)]);
                }
            }
            if (nB == 0) {
                for (int c = 0; c < nd; ++c) {
                    mbar_arrive_expect_tx(&ded_bar[c], down_bytes(c));
                    issue_down(c, ded + (size_t)c * kRingStageBytes, &ded_bar[c]);
                }
            }
            for (int k = nd; k < nC && ok; ++k) {
                const int n = nA + nB + (k - nd);
                unsigned char* dst = acquire(n, down_bytes(k));
                if (cta == 0 && k == nC - 1) trace_stamp(p.ctl, 18);
                if (dst) issue_down(k, dst, &full_bar[stage_of(n)]);
            }
        }
        if (lane == 0 && !ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingProducer);
        // Consumers wait on every full barrier that was armed, and a wait only runs out long after any
        // copy has landed, so no copy into this CTA's shared memory is in flight when the CTA leaves.
        return;
    }

    // =====================================================================================
    // Consumer warps
    // =====================================================================================
    const int group = warp / kRingGroupWarps;
    const int wi = warp % kRingGroupWarps;
    const int gtid = tid - group * kRingGroupThreads;  // thread index inside the group
    const int fg = lane >> 2, ft = lane & 3;           // MMA fragment coordinates of this lane
    float* gred = red + (size_t)group * 2 * kRingGroupWarps * 128;
    int gbuf = 0;

    // ---- phase 0: RMSNorm of the tokens into shared memory (as T) ----
    // x and the norm weight are fetched together so that the phase costs one memory round trip.
    for (int b = 0; b < p.ntok; ++b) {
        const T* xrow = x + (size_t)b * p.H;
        float f[8], g[8];
        const int k = tid * 8;
        const bool mine = k < p.H;
        uint4 xv = make_uint4(0, 0, 0, 0), wv = make_uint4(0, 0, 0, 0);
        if (mine) {
            xv = *reinterpret_cast<const uint4*>(xrow + k);
            wv = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + k);
        }
        unpack_u4<T>(xv, f);
        unpack_u4<T>(wv, g);
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
        // hidden sizes beyond one pass of the consumer threads
        for (int kk = k + kRingConsumerThreads * 8; kk < p.H; kk += kRingConsumerThreads * 8) {
            float e[8];
            unpack_u4<T>(*reinterpret_cast<const uint4*>(xrow + kk), e);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(e[i], e[i], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_red[warp] = ss;
        named_barrier(1, kRingConsumerThreads);
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kRingConsumerWarps; ++w) tot += s_red[w];
        const float rstd = 1.0f / sqrtf(tot / (float)p.H + p.eps);
        if (mine) {
            T o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(f[i], rstd), g[i]));
            *reinterpret_cast<uint4*>(xs + (size_t)b * p.H + k) = *reinterpret_cast<const uint4*>(o);
        }
        for (int kk = k + kRingConsumerThreads * 8; kk < p.H; kk += kRingConsumerThreads * 8) {
            float e[8], h[8];
            unpack_u4<T>(*reinterpret_cast<const uint4*>(xrow + kk), e);
            unpack_u4<T>(*reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + kk), h);
            T o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(e[i], rstd), h[i]));
            *reinterpret_cast<uint4*>(xs + (size_t)b * p.H + kk) = *reinterpret_cast<const uint4*>(o);
        }
        named_barrier(1, kRingConsumerThreads);
    }
    if (tracer) trace_stamp(p.ctl, 1);

    bool ok = true;

    // One stage of rows of length hidden against all tokens.  The four warps of the group split the
    // contraction, leave their 16 x 8 partial tiles in shared memory, meet at the group's barrier and
    // then every thread of the group owns one (row, column) of the summed tile.  kind: 0 router rows,
    // 1 shared (gate, up) pairs, 2 routed (gate, up) pairs of the expert with pair mask `mask`.
    // A warp whose wait ran out still walks through the barrier so that its group never hangs.
    auto consume_rows = [&](int n, int kind, int first, int count, unsigned long long mask, int i0) {
        const int stage = stage_of(n);
        bool got = ok;
        if (got) got = mbar_wait(&full_bar[stage], use_of(n) & 1, &s_abort);
        if (!got) ok = false;
        if (SC) {
            // a warp takes whole rows (router) or whole (gate, up) pairs: nothing to combine across warps
            if (got) {
                const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kRingStageBytes);
                const int nch = p.H >> 3;
                for (int r = wi; r < count; r += kRingGroupWarps) {
                    float ga[4], ua[4];
                    if (kind == 0) {
                        rows_times_tokens<T>(sbase + (size_t)r * rowH, nullptr, xs, xs + rowH, xs + 2 * rowH, xs + 3 * rowH, p.ntok, nch, lane,
                                             ga, ua);
                        if (lane == 0) {
#pragma unroll
                            for (int t = 0; t < 4; ++t)
                                if (t < p.ntok) p.logits[(size_t)t * p.E + first + r] = ga[t];
                        }
                    } else {
                        int slot[4] = {0, 0, 0, 0};
                        int nvec = p.ntok;
                        if (kind == 1) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) slot[j] = (j < p.ntok) ? j : 0;
                        } else {
                            nvec = __popcll(mask);
                            unsigned long long m = mask;
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (m) { slot[j] = __ffsll((long long)m) - 1; m &= m - 1; }
                                else slot[j] = slot[0];
                            }
                        }
                        const T* xv[4];
#pragma unroll
                        for (int j = 0; j < 4; ++j) xv[j] = xs + (size_t)((kind == 1) ? slot[j] : fdiv(slot[j], p.fd_K)) * rowH;
                        rows_times_tokens<T>(sbase + (size_t)r * rowH, sbase + (size_t)(PR + r) * rowH, xv[0], xv[1], xv[2], xv[3], nvec, nch,
                                             lane, ga, ua);
                        if (lane == 0) {
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                if (j < nvec) {
                                    const float a = silu(ga[j]) * ua[j];
                                    if (kind == 1) p.sact[(size_t)slot[j] * p.Is + first + r] = a;
                                    else p.act[(size_t)slot[j] * p.I + i0 + r] = a;
                                }
                            }
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[stage]);  // the stage has been read
            }
            return;
        }
        float* mine = gred + ((size_t)gbuf * kRingGroupWarps + wi) * 128;
        if (got) {
            const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kRingStageBytes);
            const int nrows = (kind == 0) ? count : (PR + count);
            float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            tile_times_vectors<T>(d, sbase, p.H, nrows, xs, p.H, p.ntok, p.H, wi, kRingGroupWarps, lane);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // the stage has been read
            *reinterpret_cast<float2*>(mine + fg * 8 + 2 * ft) = make_float2(d[0], d[1]);
            *reinterpret_cast<float2*>(mine + (fg + 8) * 8 + 2 * ft) = make_float2(d[2], d[3]);
        }
        named_barrier(2 + group, kRingGroupThreads);
        if (got) {
            const float* all = gred + (size_t)gbuf * kRingGroupWarps * 128;
            const int r = gtid >> 3, c = gtid & 7;
            if (r < count) {
                if (kind == 0) {
                    if (c < p.ntok) {
                        float v = 0.0f;
#pragma unroll
                        for (int w = 0; w < kRingGroupWarps; ++w) v += all[w * 128 + r * 8 + c];
                        p.logits[(size_t)c * p.E + first + r] = v;
                    }
                } else {
                    int tok = -1, slot = 0;
                    if (kind == 1) {
                        if (c < p.ntok) { tok = c; slot = c; }
                    } else if (c < __popcll(mask)) {
                        slot = nth_set_bit(mask, c);
                        tok = fdiv(slot, p.fd_K);
                    }
                    if (tok >= 0) {
                        float gsum = 0.0f, usum = 0.0f;
#pragma unroll
                        for (int w = 0; w < kRingGroupWarps; ++w) {
                            gsum += all[w * 128 + r * 8 + tok];
                            usum += all[w * 128 + (PR + r) * 8 + tok];
                        }
                        const float a = silu(gsum) * usum;
                        if (kind == 1) p.sact[(size_t)slot * p.Is + first + r] = a;
                        else p.act[(size_t)slot * p.I + i0 + r] = a;
                    }
                }
            }
        }
        gbuf ^= 1;
    };

    // ---- phase A: router rows, then shared gate+up rows ----
    unsigned bar_target = 0;
    for (int n = 0; n <= nA; ++n) {
        if (n == nA1) {
            named_barrier(1, kRingConsumerThreads);  // all logits of this CTA are written
            if (tid == 0) bar_target = barrier_arrive(p.ctl, ncta, 0);
            if (tracer) trace_stamp(p.ctl, 2);
        }
        if (n == nA) break;
        if (n % kRingGroups != group) continue;
        int first, count;
        if (n < nA1) {
            chunk_span(r0, r1, p.rows_h, mA1, n, first, count);
            consume_rows(n, 0, first, count, 0ull, 0);
        } else {
            chunk_span(s0, s1, PR, mA2, n - nA1, first, count);
            consume_rows(n, 1, first, count, 0ull, 0);
        }
        if (tracer && n == 0) trace_stamp(p.ctl, 10);
    }
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);

    // ---- wait for every CTA's logits, then select ----
    if (tracer) trace_stamp(p.ctl, 3);
    if (tid == 0) s_flag = (s_abort == 0 && barrier_wait(p.ctl, bar_target, kStatusMoeBarrier1)) ? 1 : 0;
    named_barrier(1, kRingConsumerThreads);
    if (!s_flag) {
        if (tid == 0) { s_abort = 1; s_unique = 0; }
        __syncthreads();  // (S1) releases the producer, which sees the abort flag
        return;
    }
    if (tracer) trace_stamp(p.ctl, 4);

    if (p.E > 32 * kTopkPerLane) {
        for (int i = tid; i < p.ntok * p.E; i += kRingConsumerThreads) s_logits[i] = __ldcg(p.logits + i);
        named_barrier(1, kRingConsumerThreads);
    }
    for (int b = warp; b < p.ntok; b += kRingConsumerWarps) {
        float first = 0.0f;
        if (p.E <= 32 * kTopkPerLane) {
            // each lane keeps E/32 logits in registers; a round is two warp reductions
            float v[kTopkPerLane];
#pragma unroll
            for (int j = 0; j < kTopkPerLane; ++j) {
                const int e = lane + 32 * j;
                v[j] = (e < p.E) ? __ldcg(p.logits + (size_t)b * p.E + e) : -FLT_MAX;
            }
            float mine_logit = 0.0f;
            int mine_e = 0;
            for (int r = 0; r < p.K; ++r) {
                float lb = v[0];
                int lj = 0;
#pragma unroll
                for (int j = 1; j < kTopkPerLane; ++j)
                    if (v[j] > lb) { lb = v[j]; lj = j; }
                const unsigned bits = __float_as_uint(lb);
                const unsigned key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
                const unsigned kmax = __reduce_max_sync(kFullMask, key);
                const unsigned cand = (key == kmax && lb > -FLT_MAX) ? (unsigned)(lane + 32 * lj) : 0xffffffffu;
                unsigned win = __reduce_min_sync(kFullMask, cand);
                if (win == 0xffffffffu) win = 0;  // fewer finite logits than top_k
                const unsigned kb = (kmax & 0x80000000u) ? (kmax & 0x7fffffffu) : ~kmax;
                const float best = __uint_as_float(kb);
                if ((int)(win & 31u) == lane) {
#pragma unroll
                    for (int j = 0; j < kTopkPerLane; ++j)
                        if (j == (int)(win >> 5)) v[j] = -FLT_MAX;
                }
                if (r == 0) first = best;
                if ((r & 31) == lane) { mine_logit = best; mine_e = (int)win; }
                if ((r & 31) == 31 || r == p.K - 1) {
                    const int slot = (r & ~31) + lane;  // lane l holds selection (r & ~31) + l
                    if (slot <= r) {
                        s_pair_e[b * p.K + slot] = mine_e;
                        s_pair_w[b * p.K + slot] = mine_logit;
                    }
                }
            }
        } else {
            float* lg = s_logits + (size_t)b * p.E;
            for (int r = 0; r < p.K; ++r) {
                float best = -FLT_MAX;
                int bi = INT_MAX;
                for (int e = lane; e < p.E; e += 32) {
                    const float v = lg[e];
                    if (v > best) { best = v; bi = e; }
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const float ov = __shfl_xor_sync(kFullMask, best, off);
                    const int oi = __shfl_xor_sync(kFullMask, bi, off);
                    if (oi != INT_MAX && (bi == INT_MAX || ov > best || (ov == best && oi < bi))) { best = ov; bi = oi; }
                }
                if (bi == INT_MAX) bi = 0;
                if (r == 0) first = best;
                if (lane == 0) {
                    s_pair_e[b * p.K + r] = bi;
                    s_pair_w[b * p.K + r] = best;
                    lg[bi] = -FLT_MAX;
                }
                __syncwarp();
            }
        }
        __syncwarp();
        // soft-max over the k survivors (the first one is the maximum)
        float partial = 0.0f;
        for (int r = lane; r < p.K; r += 32) {
            const float ev = expf(s_pair_w[b * p.K + r] - first);
            s_pair_w[b * p.K + r] = ev;
            partial += ev;
        }
        const float denom = warp_sum(partial);
        __syncwarp();
        for (int r = lane; r < p.K; r += 32) {
            const float w = s_pair_w[b * p.K + r] / denom;
            s_pair_w[b * p.K + r] = w;
            if (cta == 0) {
                p.indices[(size_t)b * p.K + r] = (long long)s_pair_e[b * p.K + r];
                p.route_w[(size_t)b * p.K + r] = w;
            }
        }
    }
    named_barrier(1, kRingConsumerThreads);
    // group the (token, slot) pairs by distinct local expert: the leader of a group is its lowest
    // pair index; leaders are listed in pair order
    if (warp == 0) {
        const int npair = p.ntok * p.K;
        int count = 0;
        for (int base = 0; base < npair; base += 32) {
            const int t = base + lane;
            unsigned long long m = 0ull;
            bool leader = false;
            if (t < npair) {
                const int e = s_pair_e[t];
                if (e >= p.expert_base && e < p.expert_base + p.local_experts) {
                    for (int q = 0; q < npair; ++q)
                        if (s_pair_e[q] == e) m |= 1ull << q;
                    leader = (__ffsll((long long)m) - 1) == t;
                }
            }
            const unsigned vote = __ballot_sync(kFullMask, leader);
            if (leader) {
                const int pos = count + __popc(vote & ((1u << lane) - 1u));
                s_uniq_e[pos] = s_pair_e[t];
                s_uniq_m[pos] = m;
            }
            count += __popc(vote);
        }
        if (lane == 0) s_unique = count;
    }
    __syncthreads();  // (S1) the producer starts the routed stream
    const int n_unique = s_unique;
    if (tracer) trace_stamp(p.ctl, 5);

    // ---- phase B: routed gate+up rows -> silu(g) * u per (pair, channel) ----
    const int tasks = p.I * n_unique;
    // whole chunks per CTA (a chunk never straddles two CTAs: a partial chunk costs a full stage round trip)
    const int nch_all = fdiv(tasks, p.fd_pr);
    const int t0 = fdiv(nch_all * cta, p.fd_ncta) * PR, t1 = fdiv(nch_all * (cta + 1), p.fd_ncta) * PR;
    const int nB = chunks_in(t0, t1, p.fd_pr);
    const int mB = fdiv(t0, p.fd_pr);
    for (int k = 0; k < nB; ++k) {
        const int n = nA + k;
        if (n % kRingGroups != group) continue;
        int first, count, u, i0;
        chunk_span(t0, t1, PR, mB, k, first, count);
        fdivmod(first, p.fd_I, u, i0);
        consume_rows(n, 2, first, count, s_uniq_m[u], i0);
        if (tracer && k < kRingGroups) trace_stamp(p.ctl, 11);
    }
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);

    // ---- grid barrier 2: every CTA's activations are in the scratch buffers ----
    if (tracer) trace_stamp(p.ctl, 6);
    named_barrier(1, kRingConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 0);
    if (tid == 0) {
        bool fine = (s_abort == 0);
        if (fine) {
            const unsigned target = barrier_arrive(p.ctl, ncta, 1);
            fine = barrier_wait(p.ctl, target, kStatusMoeBarrier2);
            if (fine) barrier_finish(p.ctl, ncta);
        }
        if (!fine) s_abort = 1;
        s_flag = fine ? 1 : 0;
    }
    named_barrier(1, kRingConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 7);
    if (tid == 0) cta_stamp(p.ctl, cta, 1);
    ok = (s_flag != 0);

    // ---- activations into shared memory (the token region is reused) as a high and a low half in
    //      the storage dtype: act = hi + lo to ~2^-17 relative, and both halves are MMA operands ----
    const int npairs = p.ntok * p.K;
    const size_t act_elems = (size_t)npairs * p.I + (size_t)p.ntok * p.Is;
    T* acts_lo = acts_hi + act_elems;
    float* actf = reinterpret_cast<float*>(smem + p.off_act);  // plain-FMA path: the activations stay fp32
    const size_t shared_base = (size_t)npairs * p.I;  // element offset of the shared expert's activations
    const int nC_all = (hr > 0) ? fdiv(n_unique + p.epc - 1, p.fd_epc) : 0;
    if (ok) {
        // one item = four consecutive channels of one (pair | shared token) = one 16-byte load; a
        // thread issues kActBatch loads before it touches the results
        const int q_i = p.I >> 2, q_is = p.Is >> 2;
        const int routed_items = npairs * q_i;
        const int items = routed_items + p.ntok * q_is;
        for (int base = 0; base < items; base += kRingConsumerThreads * kActBatch) {
            float4 v[kActBatch];
            long long dst[kActBatch];
#pragma unroll
            for (int q = 0; q < kActBatch; ++q) {
                const int it = base + q * kRingConsumerThreads + tid;
                dst[q] = -1;
                v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (it < routed_items) {
                    int pair, i;
                    fdivmod(it, p.fd_qi, pair, i);
                    i *= 4;
                    const int e = s_pair_e[pair];
                    if (e >= p.expert_base && e < p.expert_base + p.local_experts) {
                        v[q] = __ldcg(reinterpret_cast<const float4*>(p.act + (size_t)pair * p.I + i));
                        dst[q] = (long long)pair * p.I + i;
                    }
                } else if (it < items) {
                    const int r = it - routed_items;
                    int b, i;
                    fdivmod(r, p.fd_qis, b, i);
                    i *= 4;
                    v[q] = __ldcg(reinterpret_cast<const float4*>(p.sact + (size_t)b * p.Is + i));
                    dst[q] = (long long)shared_base + (long long)b * p.Is + i;
                }
            }
#pragma unroll
            for (int q = 0; q < kActBatch; ++q) {
                if (dst[q] >= 0) {
                    const float in[4] = {v[q].x, v[q].y, v[q].z, v[q].w};
                    if (SC) {
                        *reinterpret_cast<float4*>(actf + dst[q]) = v[q];
                        continue;
                    }
                    T hi[4], lo[4];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        hi[i] = from_float<T>(in[i]);
                        lo[i] = from_float<T>(in[i] - to_float<T>(hi[i]));
                    }
                    *reinterpret_cast<uint2*>(acts_hi + dst[q]) = *reinterpret_cast<const uint2*>(hi);
                    *reinterpret_cast<uint2*>(acts_lo + dst[q]) = *reinterpret_cast<const uint2*>(lo);
                }
            }
        }
    }
    named_barrier(1, kRingConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 8);

    // ---- phase C: down rows.  part[slot][row]: slot < npairs routed pairs, then one per token (shared).
    //      One warp contracts one expert's block of rows over the whole intermediate length. ----
    const int nC = nC_all;
    if (SC) {
        // at most two tokens in the launch (see the host side): a row meets at most two activation vectors
        const int nchI = p.I >> 3, nchIs = p.Is >> 3;
        const int ndc = min(p.nded, nC);
        const int rg = lane >> 2, t4 = lane & 3;
        // shared expert's rows: the last group, which owns the fewest routed chunks
        if (group == kRingGroups - 1 && hr > 0 && p.Is > 0) {
            bool got = ok;
            if (got) got = mbar_wait(sdown_bar, 0, &s_abort);
            if (!got) ok = false;
            if (got) {
                const float* const ap[2] = {actf + shared_base, actf + shared_base + (p.ntok > 1 ? p.Is : 0)};
                for (int r0w = 0; r0w < hr; r0w += 8 * kRingGroupWarps) {
                    const int row = r0w + wi * 8 + rg;
                    const bool live = row < hr;
                    float sv[2];
                    quad_row_dot<T, 2>(sdown_buf + (size_t)(live ? row : 0) * p.Is, ap, nchIs, t4, sv);
                    if (live && t4 == 0) {
                        part[(npairs + 0) * p.hr_max + row] = sv[0];
                        if (p.ntok > 1) part[(npairs + 1) * p.hr_max + row] = sv[1];
                    }
                }
            }
        }
        if (tracer) trace_stamp(p.ctl, 12);
        for (int k = 0; k < nC; ++k) {
            const bool own_slot = k < ndc;
            const int n = nA + nB + (k - ndc);
            if ((own_slot ? k : n) % kRingGroups != group) continue;
            const int stage = own_slot ? 0 : stage_of(n);
            const unsigned char* slot = own_slot ? ded + (size_t)k * kRingStageBytes : ring + (size_t)stage * kRingStageBytes;
            bool got = ok;
            if (got) got = own_slot ? mbar_wait(&ded_bar[k], 0, &s_abort) : mbar_wait(&full_bar[stage], use_of(n) & 1, &s_abort);
            if (!got) { ok = false; continue; }
            const bool first_chunk = tracer && k == group;
            if (first_chunk) trace_stamp(p.ctl, 13);
            if (tracer && !first_chunk) trace_stamp(p.ctl, 19);
            const int nexp = min(p.epc, n_unique - k * p.epc);
            const int ntasks = nexp * hr;  // (expert slot, row) pairs of this chunk
            for (int t0w = 0; t0w < ntasks; t0w += 8 * kRingGroupWarps) {
                const int task = t0w + wi * 8 + rg;
                const bool live = task < ntasks;
                const int tk = live ? task : 0;
                const int es = (tk >= hr) + (tk >= 2 * hr) + (tk >= 3 * hr);
                const int row = tk - es * hr;
                const unsigned long long m = s_uniq_m[k * p.epc + es];
                const int p0 = __ffsll((long long)m) - 1;
                const unsigned long long m1 = m & (m - 1);
                const int p1 = m1 ? (__ffsll((long long)m1) - 1) : p0;
                const float* const ap[2] = {actf + (size_t)p0 * p.I, actf + (size_t)p1 * p.I};
                const T* wrow = reinterpret_cast<const T*>(slot) + ((size_t)es * p.hr_max + row) * p.I;
                float sv[2];
                if (p.ntok > 1) {
                    quad_row_dot<T, 2>(wrow, ap, nchI, t4, sv);
                } else {
                    const float* const a1[1] = {ap[0]};
                    float s1[1];
                    quad_row_dot<T, 1>(wrow, a1, nchI, t4, s1);
                    sv[0] = s1[0]; sv[1] = 0.0f;
                }
                if (live && t4 == 0) {
                    part[p0 * p.hr_max + row] = sv[0];
                    if (m1) part[p1 * p.hr_max + row] = sv[1];
                }
            }
            if (first_chunk) trace_stamp(p.ctl, 20);
            __syncwarp();
            if (lane == 0 && !own_slot) mbar_arrive(&empty_bar[stage]);  // the stage has been read
        }
    } else {
    if (warp == kRingConsumerWarps - 1 && hr > 0 && p.Is > 0) {
        // shared expert: rows from the dedicated buffer, columns = tokens
        bool got = ok;
        if (got) got = mbar_wait(sdown_bar, 0, &s_abort);
        if (!got) ok = false;
        if (got) {
            float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
            const T* ch = (fg < p.ntok) ? acts_hi + shared_base + (size_t)fg * p.Is : nullptr;
            const T* cl = (fg < p.ntok) ? acts_lo + shared_base + (size_t)fg * p.Is : nullptr;
            tile_times_split_vectors<T>(d, sdown_buf, p.Is, hr, ch, cl, p.Is, lane);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = fg + ((q & 2) ? 8 : 0), col = 2 * ft + (q & 1);
                if (row < hr && col < p.ntok) part[(npairs + col) * p.hr_max + row] = d[q];
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 12);
    const int nd = min(p.nded, nC);
    // The warps of a group share a chunk: warp wi takes expert slot wi % epc and part wi / epc of the
    // intermediate length (mma.sync is slow enough that one warp per expert would make this phase
    // compute-bound); the parts meet in shared memory at the group's barrier.
    const int ks = kRingGroupWarps / p.epc;           // parts of the contraction (epc is 1, 2 or 4)
    const int eslot = wi & (p.epc - 1);
    const int kpart = wi >> ((p.epc == 4) ? 2 : (p.epc == 2 ? 1 : 0));
    const int klen = fdiv(p.I, p.fd_ks);               // multiple of 32 (checked by the host)
    for (int k = 0; k < nC; ++k) {
        // the first nd chunks sit in slots of their own (requested during the gate/up stream), the rest
        // come through the ring
        const bool own_slot = k < nd;
        const int n = nA + nB + (k - nd);
        if ((own_slot ? k : n) % kRingGroups != group) continue;
        const int stage = own_slot ? 0 : stage_of(n);
        const unsigned char* slot = own_slot ? ded + (size_t)k * kRingStageBytes : ring + (size_t)stage * kRingStageBytes;
        bool got = ok;
        if (got) got = own_slot ? mbar_wait(&ded_bar[k], 0, &s_abort) : mbar_wait(&full_bar[stage], use_of(n) & 1, &s_abort);
        if (!got) ok = false;
        const bool first_chunk = tracer && k == group;  // diagnostic stamps of the tracer's first chunk
        if (first_chunk) trace_stamp(p.ctl, 13);
        if (tracer && !first_chunk) trace_stamp(p.ctl, 19);
        const int u = k * p.epc + eslot;
        const bool work = got && u < n_unique;
        unsigned long long mask = 0ull;
        float d[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (work) {
            const T* sbase = reinterpret_cast<const T*>(slot) + (size_t)eslot * p.hr_max * p.I + (size_t)kpart * klen;
            mask = s_uniq_m[u];
            const int ncol = __popcll(mask);
            const T* ch = nullptr;
            const T* cl = nullptr;
            if (fg < ncol) {
                const int pair = nth_set_bit(mask, fg);
                ch = acts_hi + (size_t)pair * p.I + (size_t)kpart * klen;
                cl = acts_lo + (size_t)pair * p.I + (size_t)kpart * klen;
            }
            tile_times_split_vectors<T>(d, sbase, p.I, hr, ch, cl, klen, lane);
        }
        if (first_chunk) trace_stamp(p.ctl, 20);
        __syncwarp();
        if (lane == 0 && !own_slot && got) mbar_arrive(&empty_bar[stage]);  // the stage has been read
        float* mine = gred + ((size_t)gbuf * kRingGroupWarps + wi) * 128;
        if (ks > 1) {
            if (work && kpart > 0) {
                *reinterpret_cast<float2*>(mine + fg * 8 + 2 * ft) = make_float2(d[0], d[1]);
                *reinterpret_cast<float2*>(mine + (fg + 8) * 8 + 2 * ft) = make_float2(d[2], d[3]);
            }
            named_barrier(2 + group, kRingGroupThreads);  // every warp of the group walks through, whatever happened
        }
        if (first_chunk) trace_stamp(p.ctl, 21);
        if (work && kpart == 0) {
            const int ncol = __popcll(mask);
            for (int part_i = 1; part_i < ks; ++part_i) {
                const float* other = gred + ((size_t)gbuf * kRingGroupWarps + eslot + part_i * p.epc) * 128;
                const float2 lo2 = *reinterpret_cast<const float2*>(other + fg * 8 + 2 * ft);
                const float2 hi2 = *reinterpret_cast<const float2*>(other + (fg + 8) * 8 + 2 * ft);
                d[0] += lo2.x; d[1] += lo2.y; d[2] += hi2.x; d[3] += hi2.y;
            }
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int row = fg + ((q & 2) ? 8 : 0), col = 2 * ft + (q & 1);
                if (row < hr && col < ncol) part[nth_set_bit(mask, col) * p.hr_max + row] = d[q];
            }
        }
        if (first_chunk) trace_stamp(p.ctl, 22);
        gbuf ^= 1;
    }
    }  // tensor-core path
    if (tracer) trace_stamp(p.ctl, 14);
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    named_barrier(1, kRingConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 2);
    if (s_abort != 0) return;

    // ---- combine in slot order, add the residual, round once ----
    T* out = static_cast<T*>(p.out);
    const bool exchange = p.comm.world > 1;
    const unsigned step = s_step;
    for (int idx = tid; idx < p.ntok * kRingTileRows; idx += kRingConsumerThreads) {
        const int b = idx >> 4, j = idx & (kRingTileRows - 1);
        if (j >= hr) continue;
        float v = 0.0f;
        for (int k = 0; k < p.K; ++k) {
            const int pair = b * p.K + k;
            const int e = s_pair_e[pair];
            if (e >= p.expert_base && e < p.expert_base + p.local_experts) v = fmaf(s_pair_w[pair], part[pair * p.hr_max + j], v);
        }
        if (p.Is > 0) v += part[(npairs + b) * p.hr_max + j];
        const size_t o = (size_t)b * p.H + h0 + j;
        if (exchange) {
            comm_put(p.comm, step, o, v);  // this rank's share of element o, to every rank
        } else if (p.partial_out) {
            p.partial_out[o] = v;
        } else {
            if (p.add_residual) v += to_float<T>(x[o]);
            out[o] = from_float<T>(v);
        }
    }
    if (exchange) {
        // the same thread collects the ranks' shares of its elements, in rank order
        for (int idx = tid; idx < p.ntok * kRingTileRows; idx += kRingConsumerThreads) {
            const int b = idx >> 4, j = idx & (kRingTileRows - 1);
            if (j >= hr) continue;
            const size_t o = (size_t)b * p.H + h0 + j;
            float v;
            if (!comm_get_sum(p.comm, p.ctl, step, o, &v)) continue;
            if (p.add_residual) v += to_float<T>(x[o]);
            out[o] = from_float<T>(v);
        }
        // every CTA read the counter at entry, before the first grid barrier
        if (cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);
    }
    if (tracer) trace_stamp(p.ctl, 9);
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------

// Launches the streaming variant when the shapes suit it and sets *handled; otherwise leaves
// *handled false (no error) so that the caller uses the general kernel.
int moe_decode_ring_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                           bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    const int H = a->hidden, E = a->experts, K = a->top_k, I = a->intermediate, Is = a->shared_intermediate;
    if (K <= 0 || I <= 0 || H % 32 != 0 || I % 32 != 0 || Is % 32 != 0) return MK36_OK;
    int rows_h = kRingStageBytes / (H * 2);
    if (rows_h > kRingTileRows) rows_h = kRingTileRows;
    rows_h &= ~1;
    if (rows_h < 2) return MK36_OK;
    const int pr = rows_h / 2;
    if (I % pr != 0 || Is % pr != 0) return MK36_OK;  // a stage never straddles two experts
    const void* ptrs[] = {a->x, a->norm_weight, a->router_weight, a->expert_gate, a->expert_up, a->expert_down,
                          a->shared_gate, a->shared_up, a->shared_down};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const int ncta = dev->sm_count;
    const int hr_max = (H + ncta - 1) / ncta;
    if (hr_max > kRingTileRows) return MK36_OK;
    const size_t down_block = (size_t)hr_max * I * 2;  // one expert's output rows of this CTA
    if (down_block > (size_t)kRingStageBytes || (size_t)hr_max * Is * 2 > 32768) return MK36_OK;
    if ((long long)I * kRingMaxPairs * ncta >= (1ll << 31) || (long long)H * ncta >= (1ll << 31) || (long long)E * ncta >= (1ll << 31))
        return MK36_OK;  // the kernel's index arithmetic is 31-bit
    int epc = (int)(kRingStageBytes / down_block);
    if (epc > kRingGroupWarps) epc = kRingGroupWarps;
    if (epc == 3) epc = 2;  // the group's warps split into epc expert slots x (4 / epc) parts of the contraction
    if (I % (32 * (kRingGroupWarps / epc)) != 0) return MK36_OK;

    int tb = kRingMaxTokens;
    while (tb > 1 && (long long)tb * K > kRingMaxPairs) tb >>= 1;
    if ((long long)tb * K > kRingMaxPairs) return MK36_OK;
    if (a->batch < tb) {
        tb = 1;
        while (tb < a->batch) tb <<= 1;
    }

    MoeRingParams p;
    {
        const int rc = comm_params_from(comm, H, &p.comm, "moe_decode");
        if (rc != MK36_OK) return rc;
    }
    size_t off = 0;
    auto take = [&](size_t bytes, size_t align) {
        off = align_up(off, align);
        const size_t at = off;
        off += bytes;
        return (int)at;
    };
    int nstages = 0, nded = 0;
    for (; tb >= 1; tb >>= 1) {
        off = 0;
        const int pairs = tb * K;
        p.off_sdown = take((size_t)hr_max * Is * 2, 128);
        const size_t xs_bytes = (size_t)tb * H * 2;
        const size_t act_bytes = ((size_t)pairs * I + (size_t)tb * Is) * 4;  // high + low halves
        p.off_act = take(xs_bytes > act_bytes ? xs_bytes : act_bytes, 128);
        p.off_part = take((size_t)(pairs + tb) * hr_max * 4, 16);
        p.off_red = take((size_t)kRingGroups * 2 * kRingGroupWarps * 128 * 4, 16);
        p.off_logits = take(E > 32 * kTopkPerLane ? (size_t)tb * E * 4 : 16, 16);
        p.off_uniq_e = take(kRingMaxPairs * 4, 16);
        p.off_uniq_m = take(kRingMaxPairs * 8, 16);
        p.off_pair_e = take(kRingMaxPairs * 4, 16);
        p.off_pair_w = take(kRingMaxPairs * 4, 16);
        p.off_bars = take((2 * kRingMaxStages + 1 + kRingMaxDed) * 8, 16);
        p.off_ring = take(0, 128);
        const long long room = (long long)dev->max_smem_optin - (long long)off - 1024;
        nstages = (int)(room / kRingStageBytes);
        // every consumer group owns one or two stages of its own (see stage_of below); what is left over
        // becomes single-use slots for the first down-projection chunks
        const int fit = nstages;
        nstages = (nstages >= 2 * kRingGroups) ? 2 * kRingGroups : (nstages >= kRingGroups ? kRingGroups : 0);
        nded = fit - nstages;
        if (nded > kRingMaxDed) nded = kRingMaxDed;
        if (nstages > 0) break;
    }
    if (tb < 1) return MK36_OK;
    p.off_ded = p.off_ring + nstages * kRingStageBytes;
    p.nded = nded;
    const size_t smem_bytes = (size_t)p.off_ring + (size_t)(nstages + nded) * kRingStageBytes;

    const size_t scratch = align_up((size_t)tb * E * 4, 256) + align_up((size_t)tb * K * I * 4, 256) +
                           align_up((size_t)tb * (Is > 0 ? Is : 1) * 4, 256);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + scratch)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, kControlBytes + scratch);

    p.norm_w = a->norm_weight;
    p.router_w = a->router_weight;
    p.egate = a->expert_gate;
    p.eup = a->expert_up;
    p.edown = a->expert_down;
    p.sgate = a->shared_gate;
    p.sup = a->shared_up;
    p.sdown = a->shared_down;
    p.ctl = static_cast<Control*>(workspace);
    unsigned char* sc = static_cast<unsigned char*>(workspace) + kControlBytes;
    p.logits = reinterpret_cast<float*>(sc);
    sc += align_up((size_t)tb * E * 4, 256);
    p.act = reinterpret_cast<float*>(sc);
    sc += align_up((size_t)tb * K * I * 4, 256);
    p.sact = reinterpret_cast<float*>(sc);
    p.H = H; p.E = E; p.K = K; p.I = I; p.Is = Is;
    p.expert_base = a->expert_base;
    p.local_experts = a->local_experts;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    p.nstages = nstages;
    p.rows_h = rows_h;
    p.epc = epc;
    p.hr_max = hr_max;
    p.log2_depth = (nstages >= 2 * kRingGroups) ? 1 : 0;
    p.scalar = (tb <= 2 && !options().ring_mma) ? 1 : 0;
    p.fd_ncta = make_fastdiv(ncta);
    p.fd_rows_h = make_fastdiv(rows_h);
    p.fd_pr = make_fastdiv(pr);
    p.fd_I = make_fastdiv(I);
    p.fd_K = make_fastdiv(K);
    p.fd_qi = make_fastdiv(I / 4);
    p.fd_qis = make_fastdiv(Is > 0 ? Is / 4 : 1);
    p.fd_epc = make_fastdiv(epc);
    p.fd_ks = make_fastdiv(kRingGroupWarps / epc);

    const void* kernel = (a->dtype == MK36_BF16)
                             ? (p.scalar ? (const void*)moe_decode_ring_kernel<__nv_bfloat16, true> : (const void*)moe_decode_ring_kernel<__nv_bfloat16, false>)
                             : (p.scalar ? (const void*)moe_decode_ring_kernel<__half, true> : (const void*)moe_decode_ring_kernel<__half, false>);
    {
        const int rc_smem = ensure_dynamic_smem(kernel, smem_bytes);
        if (rc_smem != MK36_OK) return rc_smem;
    }
    const size_t es = 2;
    for (int b0 = 0; b0 < a->batch; b0 += tb) {
        p.ntok = (a->batch - b0 < tb) ? (a->batch - b0) : tb;
        p.x = static_cast<const unsigned char*>(a->x) + (size_t)b0 * H * es;
        p.out = a->out ? static_cast<unsigned char*>(a->out) + (size_t)b0 * H * es : nullptr;
        p.partial_out = a->partial_out ? a->partial_out + (size_t)b0 * H : nullptr;
        p.indices = reinterpret_cast<long long*>(a->indices) + (size_t)b0 * K;
        p.route_w = a->route_weights + (size_t)b0 * K;
        void* params[] = {&p};
        int rc = launch_cooperative(kernel, dim3(ncta), dim3(kRingThreads), smem_bytes, stream, params, "moe_decode(ring)");
        if (rc != MK36_OK) return rc;
    }
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
