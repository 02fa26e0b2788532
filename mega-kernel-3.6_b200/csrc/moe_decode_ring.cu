// MoE decode, streaming variant for sm_100a (2-byte dtypes, aligned shapes).
//
// Same phases and arithmetic as the general kernel in moe_decode.cu, but the weights do not go
// through registers on their way from HBM: one producer warp feeds a shared-memory ring with 1-D
// bulk copies (cp.async.bulk completing on mbarriers, no multicast) and twelve consumer warps drain
// it.  Because weight addresses depend only on the routing decision, the producer runs ahead of
// the grid barriers: router rows, shared-expert rows and the CTA's slice of shared_down are
// requested at kernel entry, before the token is even normalised, and once the top-k is known the
// routed gate/up rows and then the routed down rows are requested back to back, so the down rows
// are already in shared memory (or in flight) while the second grid barrier completes.
//
//   stream of one CTA:  [router rows][shared gate+up rows] | [routed gate+up rows][routed down rows]
//                        issued at entry                      issued after the top-k
//
// A stage is 32 KB (bulk copies under 16 KB cost bandwidth on B200).  It holds either
//   - up to `rows_h` router rows, or
//   - gate rows i..i+n and, in its second half, up rows i..i+n of one expert (n <= rows_h / 2), so
//     that one warp forms silu(gate_i . x) * (up_i . x) without a round trip through memory, or
//   - this CTA's output rows of the down projection of up to `epc` experts.
// Stage n is consumed by warp group n % 3.  Partial results per (token, slot) pair are kept apart and
// summed in slot order at the end, so the result does not depend on timing.
#include <cfloat>
#include <climits>

#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kRingConsumerWarps = 12;  // 12 + 1 producer: 13 warps are allocated as 16, i.e. 128 registers per thread
constexpr int kRingConsumerThreads = kRingConsumerWarps * 32;
constexpr int kRingThreads = kRingConsumerThreads + 32;  // + one producer warp
constexpr int kRingStageBytes = 32768;
constexpr int kRingGroups = 3;
constexpr int kRingGroupWarps = kRingConsumerWarps / kRingGroups;
constexpr int kRingMaxStages = 6;
constexpr int kRingMaxTokens = 8;
constexpr int kRingMaxPairs = 64;
constexpr int kRingXChunks = 8;  // register-resident token: hidden <= 8 * 32 * 8 = 2048
constexpr int kTopkPerLane = 8;  // register top-k: experts <= 256
constexpr int kActBatch = 4;     // 16-byte activation loads in flight per thread

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
    int rows_h;   // rows of length H per stage (pairs per stage = rows_h / 2)
    int epc;      // experts per stage in the down phase
    int hr_max;   // max output rows per CTA
    int l2_prefetch;  // 1: request the whole routed stream into L2 as soon as routing is known
    // byte offsets into dynamic shared memory
    int off_ring, off_sdown, off_act, off_part, off_logits, off_uniq_e, off_uniq_m, off_pair_e, off_pair_w, off_bars;
};

__device__ __forceinline__ int chunks_in(int r0, int r1, int per) { return r1 > r0 ? ((r1 - 1) / per - r0 / per + 1) : 0; }

// items [first, first + count) of chunk n of the range [r0, r1), chunks aligned to multiples of `per`
__device__ __forceinline__ void chunk_span(int r0, int r1, int per, int n, int& first, int& count) {
    const int m = r0 / per + n;
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

// Two rows of shared memory against the register-resident token: independent accumulation chains,
// interleaved reductions.  With two == false the second row is not read.
template <typename T>
__device__ __forceinline__ void row_dot_regs2(const T* srow0, const T* srow1, bool two, int Hc, int lane,
                                              const float (&xr)[kRingXChunks][8], float& out0, float& out1) {
    float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
#pragma unroll
    for (int j = 0; j < kRingXChunks; ++j) {
        const int c = lane + 32 * j;
        if (c < Hc) {
            float f[8], g[8];
            unpack_u4<T>(lds128(srow0 + 8 * c), f);
            unpack_u4<T>(two ? lds128(srow1 + 8 * c) : make_uint4(0, 0, 0, 0), g);
#pragma unroll
            for (int i = 0; i < 8; i += 2) {
                a0 = fmaf(f[i], xr[j][i], a0);
                a1 = fmaf(f[i + 1], xr[j][i + 1], a1);
                b0 = fmaf(g[i], xr[j][i], b0);
                b1 = fmaf(g[i + 1], xr[j][i + 1], b1);
            }
        }
    }
    float a = a0 + a1, b = b0 + b1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
        a += __shfl_xor_sync(kFullMask, a, off);
        b += __shfl_xor_sync(kFullMask, b, off);
    }
    out0 = a;
    out1 = b;
}

// Two rows of shared memory against NT tokens kept in shared memory as T (token t at xs + tok[t] * H).
template <typename T, int NT>
__device__ __forceinline__ void row_dot_smem2(const T* srow0, const T* srow1, bool two, int Hc, int lane, const T* xs,
                                              const int (&tok)[NT], int H, float (&out0)[NT], float (&out1)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) { out0[t] = 0.0f; out1[t] = 0.0f; }
    for (int c = lane; c < Hc; c += 32) {
        float f[8], g[8];
        unpack_u4<T>(lds128(srow0 + 8 * c), f);
        unpack_u4<T>(two ? lds128(srow1 + 8 * c) : make_uint4(0, 0, 0, 0), g);
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            float xv[8];
            unpack_u4<T>(lds128(xs + (size_t)tok[t] * H + 8 * c), xv);
            float s0 = out0[t], s1 = out1[t];
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                s0 = fmaf(f[i], xv[i], s0);
                s1 = fmaf(g[i], xv[i], s1);
            }
            out0[t] = s0;
            out1[t] = s1;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int t = 0; t < NT; ++t) {
            out0[t] += __shfl_xor_sync(kFullMask, out0[t], off);
            out1[t] += __shfl_xor_sync(kFullMask, out1[t], off);
        }
    }
}

// Up to R rows of shared memory (row r at base + r * row_stride elements, r < nrows) against one
// fp32 activation vector in the split layout; the R chains and reductions are interleaved.
template <typename T, int R>
__device__ __forceinline__ void rows_dot_act(const T* base, int row_stride, int nrows, const float* act, int half,
                                             int nchunks, int lane, float (&out)[R]) {
    float acc[R];
#pragma unroll
    for (int r = 0; r < R; ++r) acc[r] = 0.0f;
    for (int c = lane; c < nchunks; c += 32) {
        const float4 a = *reinterpret_cast<const float4*>(act + 4 * c);
        const float4 b = *reinterpret_cast<const float4*>(act + half + 4 * c);
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r < nrows) {
                float f[8];
                unpack_u4<T>(lds128(base + (size_t)r * row_stride + 8 * c), f);
                float s = acc[r];
                s = fmaf(f[0], a.x, s); s = fmaf(f[1], a.y, s); s = fmaf(f[2], a.z, s); s = fmaf(f[3], a.w, s);
                s = fmaf(f[4], b.x, s); s = fmaf(f[5], b.y, s); s = fmaf(f[6], b.z, s); s = fmaf(f[7], b.w, s);
                acc[r] = s;
            }
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int r = 0; r < R; ++r) acc[r] += __shfl_xor_sync(kFullMask, acc[r], off);
    }
#pragma unroll
    for (int r = 0; r < R; ++r) out[r] = acc[r];
}

// gate row and up row of one intermediate channel against the tokens listed in `mask` (bits =
// (token, slot) pair indices, or token indices when K == 0): writes silu(g) * u per listed entry.
template <typename T, int NT>
__device__ __forceinline__ void pair_rows_smem(const T* grow, const T* urow, int Hc, int H, int lane, const T* xs,
                                               unsigned long long mask, int K, float* dst, int dst_stride, int i) {
    int tok[NT], slot[NT];
    int n = 0;
    unsigned long long m = mask;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (m) {
            const int bit = __ffsll((long long)m) - 1;
            m &= m - 1;
            slot[t] = bit;
            tok[t] = K > 0 ? bit / K : bit;
            n = t + 1;
        } else {
            slot[t] = 0;
            tok[t] = 0;
        }
    }
    float g[NT], u[NT];
    row_dot_smem2<T, NT>(grow, urow, true, Hc, lane, xs, tok, H, g, u);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
            if (t < n) dst[(size_t)slot[t] * dst_stride + i] = silu(g[t]) * u[t];
    }
}

template <typename T>
__device__ __forceinline__ void pair_rows_dispatch(const T* grow, const T* urow, int Hc, int H, int lane, const T* xs,
                                                   unsigned long long mask, int K, float* dst, int dst_stride, int i) {
    const int cnt = __popcll(mask);
    if (cnt == 1) pair_rows_smem<T, 1>(grow, urow, Hc, H, lane, xs, mask, K, dst, dst_stride, i);
    else if (cnt == 2) pair_rows_smem<T, 2>(grow, urow, Hc, H, lane, xs, mask, K, dst, dst_stride, i);
    else if (cnt <= 4) pair_rows_smem<T, 4>(grow, urow, Hc, H, lane, xs, mask, K, dst, dst_stride, i);
    else pair_rows_smem<T, 8>(grow, urow, Hc, H, lane, xs, mask, K, dst, dst_stride, i);
}

// XR: the (single) token lives in registers.
template <typename T, bool XR>
__global__ void __launch_bounds__(kRingThreads, 1) moe_decode_ring_kernel(const MoeRingParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_unique;
    __shared__ int s_abort;
    __shared__ float s_red[kRingConsumerWarps];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kRingConsumerWarps);

    unsigned char* ring = smem + p.off_ring;
    T* sdown_buf = reinterpret_cast<T*>(smem + p.off_sdown);
    T* xs = reinterpret_cast<T*>(smem + p.off_act);            // phases A/B: tokens as T [ntok][H]
    float* acts = reinterpret_cast<float*>(smem + p.off_act);  // phase C: activations (split layout)
    float* part = reinterpret_cast<float*>(smem + p.off_part); // [npairs + ntok][hr_max]
    float* s_logits = reinterpret_cast<float*>(smem + p.off_logits);
    int* s_uniq_e = reinterpret_cast<int*>(smem + p.off_uniq_e);
    unsigned long long* s_uniq_m = reinterpret_cast<unsigned long long*>(smem + p.off_uniq_m);
    int* s_pair_e = reinterpret_cast<int*>(smem + p.off_pair_e);
    float* s_pair_w = reinterpret_cast<float*>(smem + p.off_pair_w);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_bar = full_bar + kRingMaxStages;
    unsigned long long* sdown_bar = empty_bar + kRingMaxStages;

    const T* x = static_cast<const T*>(p.x);
    const int NS = p.nstages;
    const int Hc = p.H >> 3;
    const size_t rowH = (size_t)p.H;       // elements per row of length hidden
    const int PR = p.rows_h >> 1;          // (gate, up) pairs per stage
    const size_t up_off = (size_t)PR * rowH;  // element offset of the up rows inside a stage

    // ---- static partition of this CTA's work ----
    const int r0 = (int)(((long long)p.E * cta) / ncta), r1 = (int)(((long long)p.E * (cta + 1)) / ncta);
    const int s0 = (int)(((long long)p.Is * cta) / ncta), s1 = (int)(((long long)p.Is * (cta + 1)) / ncta);
    const int h0 = (int)(((long long)p.H * cta) / ncta), h1 = (int)(((long long)p.H * (cta + 1)) / ncta);
    const int hr = h1 - h0;
    const int nA1 = chunks_in(r0, r1, p.rows_h);
    const int nA2 = chunks_in(s0, s1, PR);
    const int nA = nA1 + nA2;

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);
    if (tid == 0) cta_stamp(p.ctl, cta, 3);

    if (tid == 0) {
        s_abort = 0;
        for (int s = 0; s < kRingMaxStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], kRingGroupWarps);
        }
        mbar_init(sdown_bar, 1);
        mbar_init_fence();
    }
    __syncthreads();

    // =====================================================================================
    // Producer warp (one lane issues; every copy is at most one stage)
    // =====================================================================================
    if (is_producer) {
        bool ok = true;
        // chunk n goes to stage n % NS once the consumers of chunk n - NS have released it
        auto acquire = [&](int n, unsigned bytes) -> unsigned char* {
            const int stage = n % NS;
            if (n >= NS) ok = mbar_wait(&empty_bar[stage], ((n / NS) - 1) & 1, &s_abort);
            if (!ok) return nullptr;
            mbar_arrive_expect_tx(&full_bar[stage], bytes);
            return ring + (size_t)stage * kRingStageBytes;
        };
        if (lane == 0) {
            // shared_down rows of this CTA: needed only in the last phase, requested first
            if (hr > 0 && p.Is > 0) {
                const unsigned bytes = (unsigned)((size_t)hr * p.Is * sizeof(T));
                mbar_arrive_expect_tx(sdown_bar, bytes);
                bulk_copy_g2s(sdown_buf, static_cast<const T*>(p.sdown) + (size_t)h0 * p.Is, bytes, sdown_bar);
            }
            for (int n = 0; n < nA && ok; ++n) {
                int first, count;
                if (n < nA1) {
                    chunk_span(r0, r1, p.rows_h, n, first, count);
                    const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                    unsigned char* dst = acquire(n, bytes);
                    if (dst) bulk_copy_g2s(dst, static_cast<const T*>(p.router_w) + (size_t)first * rowH, bytes, &full_bar[n % NS]);
                } else {
                    chunk_span(s0, s1, PR, n - nA1, first, count);
                    const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                    unsigned char* dst = acquire(n, 2 * bytes);
                    if (dst) {
                        bulk_copy_g2s(dst, static_cast<const T*>(p.sgate) + (size_t)first * rowH, bytes, &full_bar[n % NS]);
                        bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.sup) + (size_t)first * rowH, bytes, &full_bar[n % NS]);
                    }
                }
            }
        }
        __syncthreads();  // (S1) routing is known
        const int n_unique = s_unique;
        if (s_abort != 0) ok = false;
        if (lane == 0 && ok) {
            const long long tasks = (long long)p.I * n_unique;
            const int t0 = (int)(tasks * cta / ncta), t1 = (int)(tasks * (cta + 1) / ncta);
            const int nB = chunks_in(t0, t1, PR);
            const int nC = (hr > 0) ? (n_unique + p.epc - 1) / p.epc : 0;
            // Ask for everything this CTA will stream to be brought into L2 right away: the ring
            // below can only keep a few stages in flight, and a cold HBM access (with its address
            // translation) takes microseconds, so without this the later chunks would start their
            // long trip only when a stage is released.
            if (p.l2_prefetch) {
                for (int k = 0; k < nB; ++k) {
                    int first, count;
                    chunk_span(t0, t1, PR, k, first, count);
                    const int u = first / p.I, i = first - u * p.I;
                    const size_t off = ((size_t)(s_uniq_e[u] - p.expert_base) * p.I + i) * rowH;
                    const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                    bulk_prefetch_l2(static_cast<const T*>(p.egate) + off, bytes);
                    bulk_prefetch_l2(static_cast<const T*>(p.eup) + off, bytes);
                }
                if (hr > 0) {
                    for (int u = 0; u < n_unique; ++u)
                        bulk_prefetch_l2(static_cast<const T*>(p.edown) + ((size_t)(s_uniq_e[u] - p.expert_base) * p.H + h0) * p.I,
                                         (unsigned)((size_t)hr * p.I * sizeof(T)));
                }
            }
            for (int k = 0; k < nB && ok; ++k) {
                int first, count;
                chunk_span(t0, t1, PR, k, first, count);
                const int u = first / p.I, i = first - u * p.I;
                const int e = s_uniq_e[u] - p.expert_base;
                const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                const int n = nA + k;
                unsigned char* dst = acquire(n, 2 * bytes);
                if (cta == 0 && k == 0) trace_stamp(p.ctl, 15);
                if (cta == 0 && k == nB - 1) trace_stamp(p.ctl, 16);
                if (dst) {
                    const size_t off = ((size_t)e * p.I + i) * rowH;
                    bulk_copy_g2s(dst, static_cast<const T*>(p.egate) + off, bytes, &full_bar[n % NS]);
                    bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.eup) + off, bytes, &full_bar[n % NS]);
                }
            }
            const unsigned cbytes = (unsigned)((size_t)hr * p.I * sizeof(T));
            for (int k = 0; k < nC && ok; ++k) {
                const int ua = k * p.epc, ub = min(n_unique, ua + p.epc);
                const int n = nA + nB + k;
                unsigned char* dst = acquire(n, cbytes * (unsigned)(ub - ua));
                if (cta == 0 && k == 0) trace_stamp(p.ctl, 17);
                if (cta == 0 && k == nC - 1) trace_stamp(p.ctl, 18);
                if (dst) {
                    for (int u = ua; u < ub; ++u) {
                        const int e = s_uniq_e[u] - p.expert_base;
                        bulk_copy_g2s(dst + (size_t)(u - ua) * p.hr_max * p.I * sizeof(T),
                                      static_cast<const T*>(p.edown) + ((size_t)e * p.H + h0) * p.I, cbytes, &full_bar[n % NS]);
                    }
                }
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
    float xr[kRingXChunks][8];
    if (XR) {
#pragma unroll
        for (int j = 0; j < kRingXChunks; ++j) {
            const int c = lane + 32 * j;
            if (c < Hc) {
                unpack_u4<T>(lds128(xs + 8 * c), xr[j]);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) xr[j][i] = 0.0f;
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 1);

    const unsigned long long all_tokens = (p.ntok >= 64) ? ~0ull : ((1ull << p.ntok) - 1ull);

    bool ok = true;
    // ---- phase A: router rows, then shared gate+up rows ----
    // (A warp that has given up keeps walking the loops without touching data, so that every
    // named barrier below is still reached by all consumer warps.)
    unsigned bar_target = 0;
    for (int n = 0; n <= nA; ++n) {
        if (n == nA1) {
            named_barrier(1, kRingConsumerThreads);  // all logits of this CTA are written
            if (tid == 0) bar_target = barrier_arrive(p.ctl, ncta, 0);
            if (tracer) trace_stamp(p.ctl, 2);
        }
        if (n == nA) break;
        if (n % kRingGroups != group) continue;
        const int stage = n % NS;
        if (ok) ok = mbar_wait(&full_bar[stage], (n / NS) & 1, &s_abort);
        if (!ok) continue;
        if (tracer && n == 0) trace_stamp(p.ctl, 10);
        const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kRingStageBytes);
        int first, count;
        if (n < nA1) {
            chunk_span(r0, r1, p.rows_h, n, first, count);
            for (int j = wi; j < count; j += 2 * kRingGroupWarps) {
                const bool two = (j + kRingGroupWarps) < count;
                const T* row0 = sbase + (size_t)j * rowH;
                const T* row1 = sbase + (size_t)(j + kRingGroupWarps) * rowH;
                if (XR) {
                    float v0, v1;
                    row_dot_regs2<T>(row0, row1, two, Hc, lane, xr, v0, v1);
                    if (lane == 0) {
                        p.logits[first + j] = v0;
                        if (two) p.logits[first + j + kRingGroupWarps] = v1;
                    }
                } else {
                    int tok[kRingMaxTokens];
#pragma unroll
                    for (int t = 0; t < kRingMaxTokens; ++t) tok[t] = (t < p.ntok) ? t : 0;
                    float v0[kRingMaxTokens], v1[kRingMaxTokens];
                    row_dot_smem2<T, kRingMaxTokens>(row0, row1, two, Hc, lane, xs, tok, p.H, v0, v1);
                    if (lane == 0) {
#pragma unroll
                        for (int t = 0; t < kRingMaxTokens; ++t) {
                            if (t < p.ntok) {
                                p.logits[(size_t)t * p.E + first + j] = v0[t];
                                if (two) p.logits[(size_t)t * p.E + first + j + kRingGroupWarps] = v1[t];
                            }
                        }
                    }
                }
            }
        } else {
            chunk_span(s0, s1, PR, n - nA1, first, count);
            for (int j = wi; j < count; j += kRingGroupWarps) {
                const T* grow = sbase + (size_t)j * rowH;
                const T* urow = sbase + up_off + (size_t)j * rowH;
                if (XR) {
                    float g, u;
                    row_dot_regs2<T>(grow, urow, true, Hc, lane, xr, g, u);
                    if (lane == 0) p.sact[first + j] = silu(g) * u;
                } else {
                    pair_rows_dispatch<T>(grow, urow, Hc, p.H, lane, xs, all_tokens, 0, p.sact, p.Is, first + j);
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
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
    const long long tasks = (long long)p.I * n_unique;
    const int t0 = (int)(tasks * cta / ncta), t1 = (int)(tasks * (cta + 1) / ncta);
    const int nB = chunks_in(t0, t1, PR);
    for (int k = 0; k < nB && ok; ++k) {
        const int n = nA + k;
        if (n % kRingGroups != group) continue;
        const int stage = n % NS;
        ok = mbar_wait(&full_bar[stage], (n / NS) & 1, &s_abort);
        if (!ok) break;  // no named barrier inside this loop, leaving early is safe
        if (tracer && k < kRingGroups) trace_stamp(p.ctl, 11);
        const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kRingStageBytes);
        int first, count;
        chunk_span(t0, t1, PR, k, first, count);
        const int u = first / p.I, i0 = first - u * p.I;
        const unsigned long long m = s_uniq_m[u];
        for (int j = wi; j < count; j += kRingGroupWarps) {
            const T* grow = sbase + (size_t)j * rowH;
            const T* urow = sbase + up_off + (size_t)j * rowH;
            if (XR) {
                float g, up;
                row_dot_regs2<T>(grow, urow, true, Hc, lane, xr, g, up);
                if (lane == 0) p.act[(size_t)(__ffsll((long long)m) - 1) * p.I + i0 + j] = silu(g) * up;
            } else {
                pair_rows_dispatch<T>(grow, urow, Hc, p.H, lane, xs, m, p.K, p.act, p.I, i0 + j);
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
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

    // ---- activations into shared memory (the token region is reused), split layout ----
    const int Ic = p.I >> 3, Isc = p.Is >> 3;
    const int a_half = Ic * 4, a_stride = Ic * 8;
    const int sa_half = Isc * 4, sa_stride = Isc * 8;
    const int npairs = p.ntok * p.K;
    float* sacts = acts + (size_t)npairs * a_stride;
    if (ok) {
        // one item = four consecutive channels of one (pair | shared token) = one 16-byte load; a
        // thread issues kActBatch loads before it touches the results
        const int q_i = p.I >> 2, q_is = p.Is >> 2;
        const int routed_items = npairs * q_i;
        const int items = routed_items + p.ntok * q_is;
        for (int base = 0; base < items; base += kRingConsumerThreads * kActBatch) {
            float4 v[kActBatch];
            int dst[kActBatch];
#pragma unroll
            for (int q = 0; q < kActBatch; ++q) {
                const int it = base + q * kRingConsumerThreads + tid;
                dst[q] = -1;
                v[q] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (it < routed_items) {
                    const int pair = it / q_i, i = (it - pair * q_i) * 4;
                    const int e = s_pair_e[pair];
                    if (e >= p.expert_base && e < p.expert_base + p.local_experts) {
                        v[q] = __ldcg(reinterpret_cast<const float4*>(p.act + (size_t)pair * p.I + i));
                        dst[q] = pair * a_stride + split_index(i, a_half);
                    }
                } else if (it < items) {
                    const int r = it - routed_items;
                    const int b = r / q_is, i = (r - b * q_is) * 4;
                    v[q] = __ldcg(reinterpret_cast<const float4*>(p.sact + (size_t)b * p.Is + i));
                    dst[q] = npairs * a_stride + b * sa_stride + split_index(i, sa_half);
                }
            }
#pragma unroll
            for (int q = 0; q < kActBatch; ++q)
                if (dst[q] >= 0) *reinterpret_cast<float4*>(acts + dst[q]) = v[q];
        }
    }
    named_barrier(1, kRingConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 8);

    // ---- phase C: down rows.  part[slot][row]: slot < npairs routed pairs, then one per token (shared) ----
    const int nC = (hr > 0) ? (n_unique + p.epc - 1) / p.epc : 0;
    if (ok && hr > 0 && p.Is > 0) {
        ok = mbar_wait(sdown_bar, 0, &s_abort);
        if (ok) {
            // shared expert: row j -> warp j % 12; a warp does its (up to two) rows together
            for (int j = warp; j < hr; j += 2 * kRingConsumerWarps) {
                const int nrows = (j + kRingConsumerWarps < hr) ? 2 : 1;
                for (int t = 0; t < p.ntok; ++t) {
                    float v[2];
                    rows_dot_act<T, 2>(sdown_buf + (size_t)j * p.Is, kRingConsumerWarps * p.Is, nrows, sacts + t * sa_stride, sa_half,
                                       Isc, lane, v);
                    if (lane == 0) {
                        part[(npairs + t) * p.hr_max + j] = v[0];
                        if (nrows == 2) part[(npairs + t) * p.hr_max + j + kRingConsumerWarps] = v[1];
                    }
                }
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 12);
    for (int k = 0; k < nC && ok; ++k) {
        const int n = nA + nB + k;
        if (n % kRingGroups != group) continue;
        const int stage = n % NS;
        ok = mbar_wait(&full_bar[stage], (n / NS) & 1, &s_abort);
        if (!ok) break;
        if (tracer && k < kRingGroups) trace_stamp(p.ctl, 13);
        if (tracer && k >= kRingGroups) trace_stamp(p.ctl, 19);
        const int ua = k * p.epc, ub = min(n_unique, ua + p.epc);
        for (int u = ua; u < ub; ++u) {
            const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kRingStageBytes) + (size_t)(u - ua) * p.hr_max * p.I;
            const unsigned long long mask = s_uniq_m[u];
            // rows wi + 4q of this expert's block belong to this warp; four of them are done together
            for (int j = wi; j < hr; j += 4 * kRingGroupWarps) {
                const int nrows = min(4, (hr - j + kRingGroupWarps - 1) / kRingGroupWarps);
                unsigned long long m = mask;
                while (m) {
                    const int pair = __ffsll((long long)m) - 1;
                    m &= m - 1;
                    float v[4];
                    rows_dot_act<T, 4>(sbase + (size_t)j * p.I, kRingGroupWarps * p.I, nrows, acts + pair * a_stride, a_half, Ic, lane, v);
                    if (lane == 0) {
#pragma unroll
                        for (int q = 0; q < 4; ++q)
                            if (q < nrows) part[pair * p.hr_max + j + q * kRingGroupWarps] = v[q];
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
    }
    if (tracer) trace_stamp(p.ctl, 14);
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    named_barrier(1, kRingConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 2);
    if (s_abort != 0) return;

    // ---- combine in slot order, add the residual, round once ----
    T* out = static_cast<T*>(p.out);
    for (int idx = tid; idx < p.ntok * hr; idx += kRingConsumerThreads) {
        const int b = idx / hr, j = idx - b * hr;
        float v = 0.0f;
        for (int k = 0; k < p.K; ++k) {
            const int pair = b * p.K + k;
            const int e = s_pair_e[pair];
            if (e >= p.expert_base && e < p.expert_base + p.local_experts) v = fmaf(s_pair_w[pair], part[pair * p.hr_max + j], v);
        }
        if (p.Is > 0) v += part[(npairs + b) * p.hr_max + j];
        const size_t o = (size_t)b * p.H + h0 + j;
        if (p.partial_out) {
            p.partial_out[o] = v;
        } else {
            if (p.add_residual) v += to_float<T>(x[o]);
            out[o] = from_float<T>(v);
        }
    }
    if (tracer) trace_stamp(p.ctl, 9);
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------
namespace {

template <typename T>
const void* ring_kernel_for(bool xr) {
    return xr ? (const void*)moe_decode_ring_kernel<T, true> : (const void*)moe_decode_ring_kernel<T, false>;
}

}  // namespace

// Launches the streaming variant when the shapes suit it and sets *handled; otherwise leaves
// *handled false (no error) so that the caller uses the general kernel.
int moe_decode_ring_launch(const mk36_moe_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    const int H = a->hidden, E = a->experts, K = a->top_k, I = a->intermediate, Is = a->shared_intermediate;
    if (K <= 0 || I <= 0 || H % 8 != 0 || I % 8 != 0 || Is % 8 != 0) return MK36_OK;
    const int row_h = H * 2;
    int rows_h = kRingStageBytes / row_h;
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
    const size_t down_block = (size_t)hr_max * I * 2;  // one expert's output rows of this CTA
    if (down_block > (size_t)kRingStageBytes || (size_t)hr_max * Is * 2 > 32768) return MK36_OK;
    const int epc = (int)(kRingStageBytes / down_block);

    int tb = kRingMaxTokens;
    while (tb > 1 && (long long)tb * K > kRingMaxPairs) tb >>= 1;
    if ((long long)tb * K > kRingMaxPairs) return MK36_OK;
    if (a->batch < tb) {
        tb = 1;
        while (tb < a->batch) tb <<= 1;
    }

    MoeRingParams p;
    size_t off = 0;
    auto take = [&](size_t bytes, size_t align) {
        off = align_up(off, align);
        const size_t at = off;
        off += bytes;
        return (int)at;
    };
    int nstages = 0;
    for (; tb >= 1; tb >>= 1) {
        off = 0;
        const int pairs = tb * K;
        p.off_sdown = take((size_t)hr_max * Is * 2, 128);
        const size_t xs_bytes = (size_t)tb * H * 2;
        const size_t act_bytes = ((size_t)pairs * I + (size_t)tb * Is) * 4;
        p.off_act = take(xs_bytes > act_bytes ? xs_bytes : act_bytes, 128);
        p.off_part = take((size_t)(pairs + tb) * hr_max * 4, 16);
        p.off_logits = take(E > 32 * kTopkPerLane ? (size_t)tb * E * 4 : 16, 16);
        p.off_uniq_e = take(kRingMaxPairs * 4, 16);
        p.off_uniq_m = take(kRingMaxPairs * 8, 16);
        p.off_pair_e = take(kRingMaxPairs * 4, 16);
        p.off_pair_w = take(kRingMaxPairs * 4, 16);
        p.off_bars = take((2 * kRingMaxStages + 1) * 8, 16);
        p.off_ring = take(0, 128);
        const long long room = (long long)dev->max_smem_optin - (long long)off - 1024;
        nstages = (int)(room / kRingStageBytes);
        if (nstages > kRingMaxStages) nstages = kRingMaxStages;
        if (nstages >= 3) break;
    }
    if (tb < 1) return MK36_OK;
    const size_t smem_bytes = (size_t)p.off_ring + (size_t)nstages * kRingStageBytes;

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
    p.l2_prefetch = options().l2_prefetch;

    const size_t es = 2;
    for (int b0 = 0; b0 < a->batch; b0 += tb) {
        const int ntok = (a->batch - b0 < tb) ? (a->batch - b0) : tb;
        const bool xr = (ntok == 1 && H <= kRingXChunks * 32 * 8);
        const void* kernel = (a->dtype == MK36_BF16) ? ring_kernel_for<__nv_bfloat16>(xr) : ring_kernel_for<__half>(xr);
        MK36_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes));
        p.ntok = ntok;
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
