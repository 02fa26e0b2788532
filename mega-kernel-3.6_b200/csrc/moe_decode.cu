// MoE decode for sm_100a: one persistent cooperative launch per (<= 8)-token chunk.
//
//   phase 0   every CTA normalises the chunk's tokens into shared memory (fp32 math, rounded
//             through the activation dtype, as the reference's rms_norm does)
//   phase A1  router rows are split over the grid  -> logits scratch          | arrive barrier 1
//   phase A2  shared-expert gate/up rows (independent of routing) stream while the
//             barrier completes                                             | wait barrier 1
//   select    every CTA redundantly takes the top-k of each token's logits, soft-maxes the k
//             survivors and groups the (token, slot) pairs by distinct expert
//   phase B   gate/up rows of the distinct local experts -> gate/up scratch     | barrier 2
//   phase C   rows of the down projections: out[b,h] = sum_slots w * down_e[h,:].act + shared
//             + residual
//
// Replaces the reference's cooperative kernel and its seven grid.sync() phases
// (csrc/persistent_moe_decode.cu:477-581) and follows the arithmetic of
// mega_kernel_qwen36/reference.py:16-62.  Weights are streamed exactly once with 128-bit
// no-allocate loads; each distinct expert is read once however many tokens selected it.
#include <cfloat>
#include <climits>

#include "mk36_comm.cuh"
#include "mk36_common.cuh"

namespace mk36 {

constexpr int kMoeThreads = 512;
constexpr int kMoeWarps = kMoeThreads / 32;
constexpr int kMaxTokens = 8;   // tokens per launch
constexpr int kMaxPairs = 64;   // (token, slot) pairs per launch
constexpr int kRowLoads = 8;    // 16-byte (2-byte types) loads in flight per lane per row
constexpr int kDownRows = 4;    // down-projection rows in flight per warp

struct MoeParams {
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
    float* gu;      // [ntok*K][2][I]
    float* sgu;     // [ntok][2][Is]
    int ntok, H, E, K, I, Is;
    int expert_base, local_experts, add_residual;
    int vecH, vecI, vecIs;  // rows of that length may use the 8-element vector path
    float eps;
    // dynamic shared memory layout (byte offsets)
    int off_logits, off_mask, off_uniq_e, off_uniq_m, off_pair_e, off_pair_w;
    CommParams comm;  // world > 1: the epilogue sums the ranks' partial outputs over peer memory
};

// dot products of one weight row with NT activation vectors held in shared memory (split layout)
template <typename T, int NT>
__device__ __forceinline__ void row_dot_vec(const T* __restrict__ row, int nchunks, const float* __restrict__ xs,
                                            const int (&tok_off)[NT], int half_off, int lane, float (&acc)[NT]) {
    for (int c0 = lane; c0 < nchunks; c0 += 32 * kRowLoads) {
        Chunk8<T> w[kRowLoads];
#pragma unroll
        for (int j = 0; j < kRowLoads; ++j) {
            const int c = c0 + 32 * j;
            if (c < nchunks) w[j] = load_chunk8<T>(row + 8 * (size_t)c);
            else zero_chunk8<T>(w[j]);
        }
#pragma unroll
        for (int j = 0; j < kRowLoads; ++j) {
            const int c = c0 + 32 * j;
            if (c < nchunks) {
                float f[8];
                unpack8(w[j], f);
#pragma unroll
                for (int t = 0; t < NT; ++t) {
                    const float4 a = *reinterpret_cast<const float4*>(xs + tok_off[t] + 4 * c);
                    const float4 b = *reinterpret_cast<const float4*>(xs + tok_off[t] + half_off + 4 * c);
                    float s = acc[t];
                    s = fmaf(f[0], a.x, s);
                    s = fmaf(f[1], a.y, s);
                    s = fmaf(f[2], a.z, s);
                    s = fmaf(f[3], a.w, s);
                    s = fmaf(f[4], b.x, s);
                    s = fmaf(f[5], b.y, s);
                    s = fmaf(f[6], b.z, s);
                    s = fmaf(f[7], b.w, s);
                    acc[t] = s;
                }
            }
        }
    }
}

template <typename T, int NT>
__device__ __forceinline__ void row_dot_scalar(const T* __restrict__ row, int len, const float* __restrict__ xs,
                                               const int (&tok_off)[NT], int half_off, int lane, float (&acc)[NT]) {
    for (int k = lane; k < len; k += 32) {
        const float w = to_float<T>(row[k]);
        const int idx = split_index(k, half_off);
#pragma unroll
        for (int t = 0; t < NT; ++t) acc[t] = fmaf(w, xs[tok_off[t] + idx], acc[t]);
    }
}

template <typename T, int NT>
__device__ __forceinline__ void row_dot(const T* row, int len, bool vec, const float* xs, const int (&tok_off)[NT],
                                        int half_off, int lane, float (&acc)[NT]) {
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = 0.0f;
    if (vec) row_dot_vec<T, NT>(row, len >> 3, xs, tok_off, half_off, lane, acc);
    else row_dot_scalar<T, NT>(row, len, xs, tok_off, half_off, lane, acc);
#pragma unroll
    for (int t = 0; t < NT; ++t) acc[t] = warp_sum(acc[t]);
}

// One routed row for the tokens of one distinct expert: pairs are the set bits of `mask`.
template <typename T, int NT>
__device__ __forceinline__ void routed_row(const T* row, const MoeParams& p, const float* xs, int x_stride, int half_off,
                                           unsigned long long mask, int mat, int i, int lane) {
    int tok_off[NT];
    int pair[NT];
    int n = 0;
    unsigned long long m = mask;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
        if (m) {
            const int bit = __ffsll((long long)m) - 1;
            m &= m - 1;
            pair[t] = bit;
            tok_off[t] = (bit / p.K) * x_stride;
            n = t + 1;
        } else {
            pair[t] = -1;
            tok_off[t] = 0;
        }
    }
    float acc[NT];
    row_dot<T, NT>(row, p.H, p.vecH != 0, xs, tok_off, half_off, lane, acc);
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < NT; ++t)
            if (t < n) p.gu[((size_t)pair[t] * 2 + mat) * p.I + i] = acc[t];
    }
}

template <typename T, int TB>
__global__ void __launch_bounds__(kMoeThreads, 1) moe_decode_kernel(const MoeParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_unique;
    __shared__ unsigned s_step;

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool exchange = p.comm.world > 1;
    if (tid == 0) s_step = exchange ? comm_read_step(p.comm) : 0u;

    const int Hc = (p.H + 7) >> 3;        // chunks per hidden vector
    const int x_half = Hc * 4;            // floats per half of the split layout
    const int x_stride = Hc * 8;          // floats per token
    float* xs = reinterpret_cast<float*>(smem);

    float* s_logits = reinterpret_cast<float*>(smem + p.off_logits);
    unsigned long long* s_mask = reinterpret_cast<unsigned long long*>(smem + p.off_mask);
    int* s_uniq_e = reinterpret_cast<int*>(smem + p.off_uniq_e);
    unsigned long long* s_uniq_m = reinterpret_cast<unsigned long long*>(smem + p.off_uniq_m);
    int* s_pair_e = reinterpret_cast<int*>(smem + p.off_pair_e);
    float* s_pair_w = reinterpret_cast<float*>(smem + p.off_pair_w);

    const T* x = static_cast<const T*>(p.x);
    const T* norm_w = static_cast<const T*>(p.norm_w);

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);

    // ---------------- phase 0: RMSNorm into shared memory ----------------
    for (int i = tid; i < TB * x_stride; i += kMoeThreads) xs[i] = 0.0f;
    __syncthreads();
    for (int b = warp; b < p.ntok; b += kMoeWarps) {
        const T* xr = x + (size_t)b * p.H;
        float ss = 0.0f;
        for (int k = lane; k < p.H; k += 32) {
            const float v = to_float<T>(xr[k]);
            ss = fmaf(v, v, ss);
        }
        ss = warp_sum(ss);
        const float rstd = 1.0f / sqrtf(ss / (float)p.H + p.eps);
        for (int k = lane; k < p.H; k += 32) {
            const float v = to_float<T>(xr[k]);
            const float n = __fmul_rn(__fmul_rn(v, rstd), to_float<T>(norm_w[k]));
            xs[b * x_stride + split_index(k, x_half)] = round_through<T>(n);
        }
    }
    __syncthreads();

    int all_tok[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) all_tok[t] = t * x_stride;
    if (tracer) trace_stamp(p.ctl, 1);

    // ---------------- phase A1: router logits ----------------
    unsigned bar_gen = 0;
    if (p.K > 0) {
        const int r0 = (int)(((long long)p.E * cta) / ncta);
        const int r1 = (int)(((long long)p.E * (cta + 1)) / ncta);
        const T* router = static_cast<const T*>(p.router_w);
        for (int r = r0 + warp; r < r1; r += kMoeWarps) {
            float acc[TB];
            row_dot<T, TB>(router + (size_t)r * p.H, p.H, p.vecH != 0, xs, all_tok, x_half, lane, acc);
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < TB; ++t)
                    if (t < p.ntok) p.logits[(size_t)t * p.E + r] = acc[t];
            }
        }
        __syncthreads();
        if (tid == 0) bar_gen = barrier_arrive(p.ctl, ncta, 0);
        if (tracer) trace_stamp(p.ctl, 2);
    }

    // ---------------- phase A2: shared expert gate/up rows ----------------
    {
        const int rows = 2 * p.Is;
        const int r0 = (int)(((long long)rows * cta) / ncta);
        const int r1 = (int)(((long long)rows * (cta + 1)) / ncta);
        const T* sg = static_cast<const T*>(p.sgate);
        const T* su = static_cast<const T*>(p.sup);
        for (int r = r0 + warp; r < r1; r += kMoeWarps) {
            // interleave gate_i / up_i so that neighbouring tasks touch both matrices evenly
            const int i = r >> 1, mat = r & 1;
            const T* row = (mat ? su : sg) + (size_t)i * p.H;
            float acc[TB];
            row_dot<T, TB>(row, p.H, p.vecH != 0, xs, all_tok, x_half, lane, acc);
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < TB; ++t)
                    if (t < p.ntok) p.sgu[((size_t)t * 2 + mat) * p.Is + i] = acc[t];
            }
        }
    }

    int n_unique = 0;
    if (p.K > 0) {
        // ---------------- wait barrier 1, then select ----------------
        if (tracer) trace_stamp(p.ctl, 3);
        if (tid == 0) s_flag = barrier_wait(p.ctl, bar_gen, kStatusMoeBarrier1) ? 1 : 0;
        __syncthreads();
        if (!s_flag) return;
        if (tracer) trace_stamp(p.ctl, 4);

        for (int i = tid; i < p.ntok * p.E; i += kMoeThreads) s_logits[i] = __ldcg(p.logits + i);
        for (int i = tid; i < p.E; i += kMoeThreads) s_mask[i] = 0ull;
        __syncthreads();

        for (int b = warp; b < p.ntok; b += kMoeWarps) {
            float* lg = s_logits + (size_t)b * p.E;
            float first = 0.0f;
            for (int r = 0; r < p.K; ++r) {
                float best = -FLT_MAX;
                int bi = INT_MAX;
                for (int e = lane; e < p.E; e += 32) {
                    // taken entries hold -FLT_MAX and can never win; ascending e keeps the
                    // lowest index among equal values
                    const float v = lg[e];
                    if (v > best) {
                        best = v;
                        bi = e;
                    }
                }
#pragma unroll
                for (int off = 16; off > 0; off >>= 1) {
                    const float ov = __shfl_xor_sync(kFullMask, best, off);
                    const int oi = __shfl_xor_sync(kFullMask, bi, off);
                    if (oi != INT_MAX && (bi == INT_MAX || ov > best || (ov == best && oi < bi))) {
                        best = ov;
                        bi = oi;
                    }
                }
                if (bi == INT_MAX) bi = 0;  // only reachable with fewer finite logits than top_k
                if (r == 0) first = best;
                if (lane == 0) {
                    s_pair_e[b * p.K + r] = bi;
                    s_pair_w[b * p.K + r] = best;  // logit for now
                    lg[bi] = -FLT_MAX;
                }
                __syncwarp();
            }
            // soft-max over the k survivors (max is the first one)
            float part = 0.0f;
            for (int r = lane; r < p.K; r += 32) {
                const float ev = expf(s_pair_w[b * p.K + r] - first);
                s_pair_w[b * p.K + r] = ev;
                part += ev;
            }
            const float denom = warp_sum(part);
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
        __syncthreads();
        // group pairs by distinct local expert
        for (int t = tid; t < p.ntok * p.K; t += kMoeThreads) {
            const int e = s_pair_e[t];
            if (e >= p.expert_base && e < p.expert_base + p.local_experts) atomicOr(&s_mask[e], 1ull << t);
        }
        __syncthreads();
        if (warp == 0) {
            int count = 0;
            for (int base = 0; base < p.E; base += 32) {
                const int e = base + lane;
                const unsigned long long m = (e < p.E) ? s_mask[e] : 0ull;
                const unsigned vote = __ballot_sync(kFullMask, m != 0ull);
                if (m != 0ull) {
                    const int pos = count + __popc(vote & ((1u << lane) - 1u));
                    s_uniq_e[pos] = e;
                    s_uniq_m[pos] = m;
                }
                count += __popc(vote);
            }
            if (lane == 0) s_unique = count;
        }
        __syncthreads();
        n_unique = s_unique;
        if (tracer) trace_stamp(p.ctl, 5);

        // ---------------- phase B: routed gate/up rows ----------------
        const long long rows_per_expert = 2ll * p.I;
        const long long tasks = rows_per_expert * n_unique;
        const long long t0 = tasks * cta / ncta;
        const long long t1 = tasks * (cta + 1) / ncta;
        const T* eg = static_cast<const T*>(p.egate);
        const T* eu = static_cast<const T*>(p.eup);
        for (long long t = t0 + warp; t < t1; t += kMoeWarps) {
            const int u = (int)(t / rows_per_expert);
            const int r = (int)(t - (long long)u * rows_per_expert);
            const int i = r >> 1, mat = r & 1;
            const int e = s_uniq_e[u];
            const unsigned long long m = s_uniq_m[u];
            const T* row = (mat ? eu : eg) + ((size_t)(e - p.expert_base) * p.I + i) * p.H;
            const int cnt = __popcll(m);
            if (cnt == 1) routed_row<T, 1>(row, p, xs, x_stride, x_half, m, mat, i, lane);
            else if (cnt == 2) routed_row<T, 2>(row, p, xs, x_stride, x_half, m, mat, i, lane);
            else if (cnt <= 4) routed_row<T, 4>(row, p, xs, x_stride, x_half, m, mat, i, lane);
            else routed_row<T, 8>(row, p, xs, x_stride, x_half, m, mat, i, lane);
        }
    }

    // ---------------- barrier 2 ----------------
    if (tracer) trace_stamp(p.ctl, 6);
    if (!grid_barrier(p.ctl, ncta, p.K > 0 ? 1u : 0u, kStatusMoeBarrier2, &s_flag)) return;
    if (tid == 0) barrier_finish(p.ctl, ncta);
    if (tracer) trace_stamp(p.ctl, 7);

    // ---------------- phase C: activations into shared memory ----------------
    // (the shared-memory region that held the normalised tokens is reused)
    const int Ic = (p.I + 7) >> 3, Isc = (p.Is + 7) >> 3;
    const int a_half = Ic * 4, a_stride = Ic * 8;
    const int sa_half = Isc * 4, sa_stride = Isc * 8;
    const int npairs = p.ntok * p.K;
    float* acts = xs;                                  // [npairs][a_stride]
    float* sacts = xs + (size_t)npairs * a_stride;     // [ntok][sa_stride]
    for (int idx = tid; idx < npairs * a_stride; idx += kMoeThreads) acts[idx] = 0.0f;
    for (int idx = tid; idx < p.ntok * sa_stride; idx += kMoeThreads) sacts[idx] = 0.0f;
    __syncthreads();
    for (int u = 0; u < n_unique; ++u) {
        unsigned long long m = s_uniq_m[u];
        while (m) {
            const int pair = __ffsll((long long)m) - 1;
            m &= m - 1;
            const float* g = p.gu + (size_t)pair * 2 * p.I;
            for (int i = tid; i < p.I; i += kMoeThreads)
                acts[pair * a_stride + split_index(i, a_half)] = silu(__ldcg(g + i)) * __ldcg(g + p.I + i);
        }
    }
    for (int b = 0; b < p.ntok; ++b) {
        const float* g = p.sgu + (size_t)b * 2 * p.Is;
        for (int i = tid; i < p.Is; i += kMoeThreads)
            sacts[b * sa_stride + split_index(i, sa_half)] = silu(__ldcg(g + i)) * __ldcg(g + p.Is + i);
    }
    __syncthreads();
    if (tracer) trace_stamp(p.ctl, 8);

    // ---------------- phase C: down projections ----------------
    {
        const int h0 = (int)(((long long)p.H * cta) / ncta);
        const int h1 = (int)(((long long)p.H * (cta + 1)) / ncta);
        const T* ed = static_cast<const T*>(p.edown);
        const T* sd = static_cast<const T*>(p.sdown);
        T* out = static_cast<T*>(p.out);
        for (int h = h0 + warp; h < h1; h += kMoeWarps) {
            float acc[TB];
#pragma unroll
            for (int t = 0; t < TB; ++t) acc[t] = 0.0f;

            if (p.vecI) {
                // routed experts, kDownRows rows in flight
                for (int u0 = 0; u0 < n_unique; u0 += kDownRows) {
                    for (int c = lane; c < Ic; c += 32) {
                        Chunk8<T> w[kDownRows];
#pragma unroll
                        for (int j = 0; j < kDownRows; ++j) {
                            if (u0 + j < n_unique) {
                                const int e = s_uniq_e[u0 + j] - p.expert_base;
                                w[j] = load_chunk8<T>(ed + ((size_t)e * p.H + h) * p.I + 8 * (size_t)c);
                            } else {
                                zero_chunk8<T>(w[j]);
                            }
                        }
#pragma unroll
                        for (int j = 0; j < kDownRows; ++j) {
                            if (u0 + j < n_unique) {
                                float f[8];
                                unpack8(w[j], f);
                                unsigned long long m = s_uniq_m[u0 + j];
                                while (m) {
                                    const int pair = __ffsll((long long)m) - 1;
                                    m &= m - 1;
                                    const float4 a = *reinterpret_cast<const float4*>(acts + pair * a_stride + 4 * c);
                                    const float4 b = *reinterpret_cast<const float4*>(acts + pair * a_stride + a_half + 4 * c);
                                    float s = f[0] * a.x;
                                    s = fmaf(f[1], a.y, s);
                                    s = fmaf(f[2], a.z, s);
                                    s = fmaf(f[3], a.w, s);
                                    s = fmaf(f[4], b.x, s);
                                    s = fmaf(f[5], b.y, s);
                                    s = fmaf(f[6], b.z, s);
                                    s = fmaf(f[7], b.w, s);
                                    s *= s_pair_w[pair];
                                    const int tok = pair / p.K;
#pragma unroll
                                    for (int t = 0; t < TB; ++t)
                                        if (t == tok) acc[t] += s;
                                }
                            }
                        }
                    }
                }
            } else {
                for (int u = 0; u < n_unique; ++u) {
                    const int e = s_uniq_e[u] - p.expert_base;
                    const T* row = ed + ((size_t)e * p.H + h) * p.I;
                    unsigned long long m = s_uniq_m[u];
                    while (m) {
                        const int pair = __ffsll((long long)m) - 1;
                        m &= m - 1;
                        float s = 0.0f;
                        for (int i = lane; i < p.I; i += 32)
                            s = fmaf(to_float<T>(row[i]), acts[pair * a_stride + split_index(i, a_half)], s);
                        s *= s_pair_w[pair];
                        const int tok = pair / p.K;
#pragma unroll
                        for (int t = 0; t < TB; ++t)
                            if (t == tok) acc[t] += s;
                    }
                }
            }

            // shared expert
            {
                const T* row = sd + (size_t)h * p.Is;
                if (p.vecIs) {
                    for (int c0 = lane; c0 < Isc; c0 += 32 * kDownRows) {
                        Chunk8<T> w[kDownRows];
#pragma unroll
                        for (int j = 0; j < kDownRows; ++j) {
                            const int c = c0 + 32 * j;
                            if (c < Isc) w[j] = load_chunk8<T>(row + 8 * (size_t)c);
                            else zero_chunk8<T>(w[j]);
                        }
#pragma unroll
                        for (int j = 0; j < kDownRows; ++j) {
                            const int c = c0 + 32 * j;
                            if (c < Isc) {
                                float f[8];
                                unpack8(w[j], f);
#pragma unroll
                                for (int t = 0; t < TB; ++t) {
                                    const float4 a = *reinterpret_cast<const float4*>(sacts + t * sa_stride + 4 * c);
                                    const float4 b = *reinterpret_cast<const float4*>(sacts + t * sa_stride + sa_half + 4 * c);
                                    float s = acc[t];
                                    s = fmaf(f[0], a.x, s);
                                    s = fmaf(f[1], a.y, s);
                                    s = fmaf(f[2], a.z, s);
                                    s = fmaf(f[3], a.w, s);
                                    s = fmaf(f[4], b.x, s);
                                    s = fmaf(f[5], b.y, s);
                                    s = fmaf(f[6], b.z, s);
                                    s = fmaf(f[7], b.w, s);
                                    acc[t] = s;
                                }
                            }
                        }
                    }
                } else {
                    for (int i = lane; i < p.Is; i += 32) {
                        const float w = to_float<T>(row[i]);
                        const int idx = split_index(i, sa_half);
#pragma unroll
                        for (int t = 0; t < TB; ++t)
                            if (t < p.ntok) acc[t] = fmaf(w, sacts[t * sa_stride + idx], acc[t]);
                    }
                }
            }

#pragma unroll
            for (int t = 0; t < TB; ++t) acc[t] = warp_sum(acc[t]);
            if (lane == 0) {
#pragma unroll
                for (int t = 0; t < TB; ++t) {
                    if (t < p.ntok) {
                        if (exchange) {
                            comm_put(p.comm, s_step, (size_t)t * p.H + h, acc[t]);
                        } else if (p.partial_out) {
                            p.partial_out[(size_t)t * p.H + h] = acc[t];
                        } else {
                            float v = acc[t];
                            if (p.add_residual) v += to_float<T>(x[(size_t)t * p.H + h]);
                            out[(size_t)t * p.H + h] = from_float<T>(v);
                        }
                    }
                }
            }
        }
    }
    __syncthreads();
    if (exchange) {
        // collect the ranks' shares of this CTA's rows, in rank order (each element is its own flag)
        const unsigned step = s_step;
        const int h0 = (int)(((long long)p.H * cta) / ncta);
        const int h1 = (int)(((long long)p.H * (cta + 1)) / ncta);
        T* out = static_cast<T*>(p.out);
        for (int t = 0; t < p.ntok; ++t) {
            for (int h = h0 + tid; h < h1; h += kMoeThreads) {
                const size_t o = (size_t)t * p.H + h;
                float v;
                if (!comm_get_sum(p.comm, p.ctl, step, o, &v)) continue;
                if (p.add_residual) v += to_float<T>(x[o]);
                out[o] = from_float<T>(v);
            }
        }
        // every CTA read the counter at entry, before the grid barrier
        if (cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);
    }
    if (tracer) trace_stamp(p.ctl, 9);
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------
namespace {

struct MoePlan {
    int tokens_per_launch;
    size_t smem_bytes;
    size_t scratch_bytes;  // beyond the control block
    int off_logits, off_mask, off_uniq_e, off_uniq_m, off_pair_e, off_pair_w;
};

size_t elem_size(int dtype) { return dtype == MK36_F32 ? 4 : 2; }

bool plan_moe(const mk36_moe_args& a, int max_smem, MoePlan* plan) {
    const int Hc = (a.hidden + 7) / 8, Ic = (a.intermediate + 7) / 8, Isc = (a.shared_intermediate + 7) / 8;
    for (int tb = kMaxTokens; tb >= 1; tb >>= 1) {
        const long long pairs = (long long)tb * a.top_k;
        if (pairs > kMaxPairs) continue;
        size_t region = (size_t)tb * Hc * 8 * 4;
        const size_t region_c = ((size_t)pairs * Ic * 8 + (size_t)tb * Isc * 8) * 4;
        if (region_c > region) region = region_c;
        size_t off = align_up(region, 16);
        plan->off_logits = (int)off;  off += align_up((size_t)tb * a.experts * 4, 16);
        plan->off_mask = (int)off;    off += align_up((size_t)a.experts * 8, 16);
        plan->off_uniq_e = (int)off;  off += kMaxPairs * 4;
        plan->off_uniq_m = (int)off;  off += kMaxPairs * 8;
        plan->off_pair_e = (int)off;  off += kMaxPairs * 4;
        plan->off_pair_w = (int)off;  off += kMaxPairs * 4;
        if (off + 1024 > (size_t)max_smem) continue;
        plan->tokens_per_launch = tb;
        plan->smem_bytes = off;
        plan->scratch_bytes = align_up((size_t)tb * a.experts * 4, 256) +
                              align_up((size_t)(pairs > 0 ? pairs : 1) * 2 * (a.intermediate > 0 ? a.intermediate : 1) * 4, 256) +
                              align_up((size_t)tb * 2 * a.shared_intermediate * 4, 256);
        return true;
    }
    return false;
}

int check_moe_args(const mk36_moe_args* a) {
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: args is NULL");
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16 && a->dtype != MK36_F32)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "moe_decode: unsupported dtype %d", a->dtype);
    if (a->batch <= 0 || a->hidden <= 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: batch and hidden must be positive");
    if (a->experts < 0 || a->top_k < 0 || a->intermediate < 0 || a->shared_intermediate < 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: negative size");
    if (a->top_k > a->experts) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: top_k must be in [1, experts]");
    if ((a->experts > 0) != (a->top_k > 0)) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: top_k must be in [1, experts]");
    if (a->top_k > kMaxPairs) MK36_FAIL(MK36_ERR_UNSUPPORTED, "moe_decode: top_k > %d is not supported", kMaxPairs);
    if (!a->x || !a->norm_weight) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: x / norm_weight is NULL");
    if (!a->out && !a->partial_out) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: out and partial_out are both NULL");
    if (a->top_k > 0) {
        if (!a->router_weight || !a->indices || !a->route_weights)
            MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: router_weight / indices / route_weights is NULL");
        if (a->intermediate <= 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: intermediate must be positive");
        if (a->expert_base < 0 || a->local_experts < 0 || a->expert_base + a->local_experts > a->experts)
            MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: local expert range [%d, %d) outside [0, %d)", a->expert_base,
                      a->expert_base + a->local_experts, a->experts);
        if (a->local_experts > 0 && (!a->expert_gate || !a->expert_up || !a->expert_down))
            MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: expert weight pointer is NULL");
    }
    if (a->shared_intermediate > 0 && (!a->shared_gate || !a->shared_up || !a->shared_down))
        MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: shared expert weight pointer is NULL");
    return MK36_OK;
}

bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

template <typename T>
const void* moe_kernel_for(int tb) {
    switch (tb) {
        case 1: return (const void*)moe_decode_kernel<T, 1>;
        case 2: return (const void*)moe_decode_kernel<T, 2>;
        case 4: return (const void*)moe_decode_kernel<T, 4>;
        default: return (const void*)moe_decode_kernel<T, 8>;
    }
}

const void* moe_kernel(int dtype, int tb) {
    if (dtype == MK36_BF16) return moe_kernel_for<__nv_bfloat16>(tb);
    if (dtype == MK36_F16) return moe_kernel_for<__half>(tb);
    return moe_kernel_for<float>(tb);
}

}  // namespace

int moe_decode_ring_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                           bool* handled);
int moe_decode_stream_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                             bool* handled);
int moe_decode_batch_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                            bool* handled);

// `comm` (may be null) makes the kernels end with the cross-GPU sum of the ranks' partial outputs.
int moe_decode_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int rc = check_moe_args(a);
    if (rc != MK36_OK) return rc;
    if (comm && comm->world > 1 && (!a->out || a->partial_out))
        MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode: the multi-GPU entry points write `out` and take no partial_out");
    if (!options().force_generic) {
        bool handled = false;
        // one token: the stream kernel (latency-tuned); more: the batch kernel, which at two tokens is already the
        // faster of the two (34.9 against 40.1 us at the 35B shape)
        if (a->batch <= options().moe_stream && !options().ring_mma) {
            rc = moe_decode_stream_launch(a, comm, workspace, workspace_bytes, stream, &handled);
            if (rc != MK36_OK || handled) return rc;
        }
        if (options().moe_batch && !options().ring_mma) {
            rc = moe_decode_batch_launch(a, comm, workspace, workspace_bytes, stream, &handled);
            if (rc != MK36_OK || handled) return rc;
        }
        rc = moe_decode_ring_launch(a, comm, workspace, workspace_bytes, stream, &handled);
        if (rc != MK36_OK || handled) return rc;
    }
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    MoePlan plan;
    if (!plan_moe(*a, dev->max_smem_optin, &plan))
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "moe_decode: shapes do not fit in shared memory (hidden %d, intermediate %d, shared %d, top_k %d)",
                  a->hidden, a->intermediate, a->shared_intermediate, a->top_k);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + plan.scratch_bytes)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace too small (%zu < %zu bytes)", workspace_bytes,
                  kControlBytes + plan.scratch_bytes);

    const size_t es = elem_size(a->dtype);
    const int per8 = 8;
    MoeParams p;
    rc = comm_params_from(comm, a->hidden, &p.comm, "moe_decode");
    if (rc != MK36_OK) return rc;
    p.norm_w = a->norm_weight;
    p.router_w = a->router_weight;
    p.egate = a->expert_gate;
    p.eup = a->expert_up;
    p.edown = a->expert_down;
    p.sgate = a->shared_gate;
    p.sup = a->shared_up;
    p.sdown = a->shared_down;
    p.ctl = static_cast<Control*>(workspace);
    unsigned char* scratch = static_cast<unsigned char*>(workspace) + kControlBytes;
    const int tbmax = plan.tokens_per_launch;
    p.logits = reinterpret_cast<float*>(scratch);
    scratch += align_up((size_t)tbmax * a->experts * 4, 256);
    p.gu = reinterpret_cast<float*>(scratch);
    scratch += align_up((size_t)(tbmax * a->top_k > 0 ? tbmax * a->top_k : 1) * 2 * (a->intermediate > 0 ? a->intermediate : 1) * 4, 256);
    p.sgu = reinterpret_cast<float*>(scratch);
    p.H = a->hidden;
    p.E = a->experts;
    p.K = a->top_k;
    p.I = a->intermediate;
    p.Is = a->shared_intermediate;
    p.expert_base = a->expert_base;
    p.local_experts = a->local_experts;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    p.vecH = (a->hidden % per8 == 0) && aligned16(a->router_weight) && aligned16(a->expert_gate) && aligned16(a->expert_up) &&
             aligned16(a->shared_gate) && aligned16(a->shared_up);
    p.vecI = (a->intermediate % per8 == 0) && aligned16(a->expert_down);
    p.vecIs = (a->shared_intermediate % per8 == 0) && aligned16(a->shared_down);
    p.off_logits = plan.off_logits;
    p.off_mask = plan.off_mask;
    p.off_uniq_e = plan.off_uniq_e;
    p.off_uniq_m = plan.off_uniq_m;
    p.off_pair_e = plan.off_pair_e;
    p.off_pair_w = plan.off_pair_w;

    for (int b0 = 0; b0 < a->batch; b0 += tbmax) {
        const int ntok = (a->batch - b0 < tbmax) ? (a->batch - b0) : tbmax;
        int tb = 1;
        while (tb < ntok) tb <<= 1;
        const void* kernel = moe_kernel(a->dtype, tb);
        rc = ensure_dynamic_smem(kernel, plan.smem_bytes);
        if (rc != MK36_OK) return rc;
        p.ntok = ntok;
        p.x = static_cast<const unsigned char*>(a->x) + (size_t)b0 * a->hidden * es;
        p.out = a->out ? static_cast<unsigned char*>(a->out) + (size_t)b0 * a->hidden * es : nullptr;
        p.partial_out = a->partial_out ? a->partial_out + (size_t)b0 * a->hidden : nullptr;
        p.indices = a->indices ? reinterpret_cast<long long*>(a->indices) + (size_t)b0 * a->top_k : nullptr;
        p.route_w = a->route_weights ? a->route_weights + (size_t)b0 * a->top_k : nullptr;
        void* params[] = {&p};
        rc = launch_cooperative(kernel, dim3(dev->sm_count), dim3(kMoeThreads), plan.smem_bytes, stream, params, "moe_decode");
        if (rc != MK36_OK) return rc;
    }
    return MK36_OK;
}

}  // namespace mk36

using namespace mk36;

extern "C" {

size_t mk36_moe_workspace_bytes(const mk36_moe_args* a) {
    if (!a) return 0;
    MoePlan plan;
    if (!plan_moe(*a, 227 * 1024, &plan)) return 0;
    size_t need = kControlBytes + plan.scratch_bytes;
    // 2-byte dtypes use the stream kernel (one token) or the batch kernel when the workspace also holds their mailboxes
    if (a->dtype != MK36_F32 && need < kTaggedEnd) need = kTaggedEnd;
    return need;
}

int mk36_moe_decode(const mk36_moe_args* args, void* workspace, size_t workspace_bytes, void* stream) {
    return moe_decode_launch(args, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int mk36_moe_decode_ep(const mk36_moe_args* args, const mk36_comm* comm, void* workspace, size_t workspace_bytes, void* stream) {
    if (!comm) MK36_FAIL(MK36_ERR_INVALID_ARG, "moe_decode_ep: comm is NULL");
    return moe_decode_launch(args, comm, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
