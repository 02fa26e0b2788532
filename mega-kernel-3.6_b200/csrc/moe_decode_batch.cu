// MoE decode for launches of two to eight tokens on sm_100a (2-byte dtypes, aligned shapes): one
// launch, one grid barrier, one weight stream.  Same results as the general kernel in moe_decode.cu
// (reference semantics: mega_kernel_qwen36/reference.py:16-62; the reference's CUDA kernel,
// csrc/persistent_moe_decode.cu:477-581, takes the tokens of a step through seven grid-synchronised
// phases).  Eight tokens with eight experts each touch about 57 distinct experts of 256, i.e. 340 MB
// of weights: the step is a bandwidth problem with a fixed latency in front of it, and what this
// kernel does is pay that latency once for all tokens instead of once per pair of tokens.
//
//   consumers (12 warps)                                   producer warp
//   --------------------------------------------------     -------------------------------------------
//   x of all tokens, norm weight and this CTA's router      shared-expert gate/up rows and this CTA's rows
//   rows in one memory round trip; RMSNorm; router dot       of shared_down are requested at entry
//   products; every logit into every CTA's mailbox as
//   a tagged 64-bit word
//   warp b < tokens: polls the mailbox for token b's
//   logits, top-k and soft-max in registers  ------------>  groups the (token, slot) pairs by distinct
//   shared-expert (gate, up) pairs from the ring             expert; deals the routed gate/up chunks
//   routed (gate, up) pairs from the ring, against the       through the work counter; an end mark; then
//   one to eight tokens that chose the expert                this CTA's rows of every distinct expert's
//   silu(g) * u -> global scratch                            down matrix, two experts per stage, as the
//   grid barrier (the only one)                              stages come free (they do not depend on the
//   shared expert's down rows (two of three groups)          barrier: the first ones are in flight while
//   down chunks: the owning group's four warps split         the CTA waits at it)
//   the chunk's rows; the activations come from the
//   scratch (L2) straight into registers, requested
//   before the warp waits for the chunk
//   combine in slot order, residual, store / exchange
//
// Ring protocol, chunk descriptors and the rule that every consumer warp observes and releases every
// chunk are those of moe_decode_stream.cu.
#include "mk36_moe_stream.cuh"

namespace mk36 {

constexpr int kBtMaxTokens = 8;
constexpr int kBtMaxPublish = 24;  // (router row, token) logits one CTA publishes
constexpr int kBtPairStride = 8;   // pair (token b, slot r) has index b * 8 + r whatever top_k is: the token of a pair is a shift away
constexpr int kBtRowBatch = 7;     // down rows a warp keeps in flight: 14 rows per CTA split between two warps

// Token b's routing, by one warp: waits for the token's logits in this CTA's mailbox (a word is valid
// when it carries `tag`), then top-k (descending logit, lowest index on ties) and soft-max over the k
// survivors.  Writes pair_e / pair_w [b * K ..] (shared memory) and, from CTA 0, the indices and
// weights the caller asked for.  False when the wait ran out (status and abort flag are then set).
struct RouteArgs {
    const unsigned long long* box;  // this CTA's mailbox
    Control* ctl;
    long long* indices;  // null unless this CTA reports the routing
    float* route_w;
    unsigned long long* emask;  // shared memory, per expert, bit b * 8 + r: token b chose it in slot r (each byte has one writer)
    int E, K;
    int expert_base, local_experts;
};
__device__ __noinline__ bool route_token(const RouteArgs p, int b, unsigned tag, int* pair_e, float* pair_w, volatile int* abort_flag, int lane) {
    unsigned k8[kStTopkPerLane];
    unsigned spins = 0;
    {
        const unsigned long long* box = p.box + (size_t)b * p.E;
        unsigned long long t0 = 0ull;  // the wait's clock starts at the first slow check: reading the timer is not free
        unsigned have = 0u;
        for (;;) {
            bool ready = true;
#pragma unroll
            for (int j = 0; j < kStTopkPerLane; ++j) {
                const int e = lane + 32 * j;
                if (e < p.E) {
                    if (!(have & (1u << j))) {
                        const unsigned long long w = ld_relaxed_u64(box + e);
                        if ((unsigned)(w >> 32) == tag) {
                            have |= 1u << j;
                            const unsigned bits = (unsigned)w;
                            k8[j] = topk_key(bits);
                        } else {
                            ready = false;
                        }
                    }
                } else {
                    k8[j] = 0u;
                }
            }
            if (__all_sync(kFullMask, ready)) break;
            if ((++spins & 15u) == 0u) {
                bool give_up = false;
                if (lane == 0) {
                    const unsigned long long now = global_timer_ns();
                    if (t0 == 0ull) t0 = now;
                    if (*abort_flag != 0) give_up = true;
                    else if (now - t0 > kWaitLimitNs) {
                        atomicCAS(&p.ctl->status, 0, kStatusMoeLogits);
                        *abort_flag = 1;
                        give_up = true;
                    }
                }
                if (__shfl_sync(kFullMask, give_up ? 1 : 0, 0)) return false;
            }
        }
    }
    if (b == 0 && lane == 0) cta_stamp(p.ctl, blockIdx.x, 5);
    topk_select(k8, p.K, lane, [&](int r, int e, float logit) {
        pair_e[b * kBtPairStride + r] = e;
        pair_w[b * kBtPairStride + r] = logit;
        if (e >= p.expert_base && e < p.expert_base + p.local_experts) reinterpret_cast<unsigned char*>(p.emask)[e * 8 + b] = (unsigned char)(1u << r);
    });
    __syncwarp();
    const float first = pair_w[b * kBtPairStride];
    const float ev = (lane < p.K) ? expf(pair_w[b * kBtPairStride + lane] - first) : 0.0f;
    const float denom = warp_sum(ev);
    if (lane < p.K) {
        const float w = ev / denom;
        pair_w[b * kBtPairStride + lane] = w;
        if (p.indices) p.indices[(size_t)b * p.K + lane] = (long long)pair_e[b * kBtPairStride + lane];
        if (p.route_w) p.route_w[(size_t)b * p.K + lane] = w;
    }
    __syncwarp();
    return true;
}

// One or two fp32 activation vectors (global scratch, written by other CTAs before the grid barrier)
// into registers: lane l gets the 8-value pieces l and l + 32 of each.
template <int NV>
__device__ __forceinline__ void load_acts(const float* g0, const float* g1, int nchunks, int lane, float (&a)[2][2][8]) {
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        const float* ap = (t == 0) ? g0 : g1;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int c = lane + 32 * q;
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (c < nchunks) {
                v0 = __ldcg(reinterpret_cast<const float4*>(ap + 8 * c));
                v1 = __ldcg(reinterpret_cast<const float4*>(ap + 8 * c + 4));
            }
            a[t][q][0] = v0.x; a[t][q][1] = v0.y; a[t][q][2] = v0.z; a[t][q][3] = v0.w;
            a[t][q][4] = v1.x; a[t][q][5] = v1.y; a[t][q][6] = v1.z; a[t][q][7] = v1.w;
        }
    }
}

// Rows [r_begin, r_end) (at most kBtRowBatch) of a down block in shared memory (rows of `nchunks`
// 16-byte pieces, nchunks <= 64) against one or two activation vectors held in registers.  Lane l reads
// piece l and l + 32 of every row (conflict-free); all rows of the batch are in flight together.
template <typename T, int NV>
__device__ __forceinline__ void down_batch(const T* blk, int r_begin, int r_end, int nchunks, const float (&a)[2][2][8], float* out0,
                                           float* out1, int lane) {
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 w0[kBtRowBatch], w1[kBtRowBatch];
#pragma unroll
    for (int j = 0; j < kBtRowBatch; ++j) {
        const int r = r_begin + j;
        const T* w = blk + (size_t)r * nchunks * 8;
        w0[j] = (r < r_end && lane < nchunks) ? lds128(w + 8 * lane) : zero;
        w1[j] = (r < r_end && lane + 32 < nchunks) ? lds128(w + 8 * (lane + 32)) : zero;
    }
    float sv[NV][kBtRowBatch];
#pragma unroll
    for (int j = 0; j < kBtRowBatch; ++j) {
        float f0[8], f1[8];
        st_unpack<T>(w0[j], f0);
        st_unpack<T>(w1[j], f1);
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            float v0 = 0.0f, v1 = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                v0 = fmaf(f0[i], a[t][0][i], v0);
                v1 = fmaf(f1[i], a[t][1][i], v1);
            }
            sv[t][j] = v0 + v1;
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int t = 0; t < NV; ++t)
#pragma unroll
            for (int j = 0; j < kBtRowBatch; ++j) sv[t][j] += __shfl_xor_sync(kFullMask, sv[t][j], off);
    }
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < kBtRowBatch; ++j) {
            const int r = r_begin + j;
            if (r < r_end) {
                out0[r] = sv[0][j];
                if (NV > 1) out1[r] = sv[NV - 1][j];
            }
        }
    }
}

// Rows [lo, hi) of one block against the activation vectors named by the bits of `m`: bit q stands for
// the vector at abase + q * len and the partial sums at pbase + q * hr_max.  `a` already holds the
// first one or two of them when `preloaded`.
template <typename T>
__device__ __forceinline__ void down_block_rows(const T* blk, int lo, int hi, int nch, unsigned long long m, const float* abase, int len,
                                             float* pbase, int hr_max, bool preloaded, float (&a)[2][2][8], int lane) {
    bool have = preloaded;
    while (m) {
        const int q0 = __ffsll((long long)m) - 1;
        m &= m - 1;
        int q1 = -1;
        if (m) {
            q1 = __ffsll((long long)m) - 1;
            m &= m - 1;
        }
        if (q1 >= 0) {
            if (!have) load_acts<2>(abase + (size_t)q0 * len, abase + (size_t)q1 * len, nch, lane, a);
#pragma unroll 1
            for (int r = lo; r < hi; r += kBtRowBatch)
                down_batch<T, 2>(blk, r, min(hi, r + kBtRowBatch), nch, a, pbase + q0 * hr_max, pbase + q1 * hr_max, lane);
        } else {
            if (!have) load_acts<1>(abase + (size_t)q0 * len, abase, nch, lane, a);
#pragma unroll 1
            for (int r = lo; r < hi; r += kBtRowBatch) down_batch<T, 1>(blk, r, min(hi, r + kBtRowBatch), nch, a, pbase + q0 * hr_max, pbase, lane);
        }
        have = false;
    }
}

template <typename T>
__global__ void __launch_bounds__(kStThreads, 1) moe_decode_batch_kernel(const MoeStreamParams p) {
    constexpr int NT = kBtMaxTokens;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_unique;
    __shared__ int s_abort;
    __shared__ unsigned s_step;
    __shared__ unsigned s_epoch;
    __shared__ float s_red[kStConsumerWarps][NT];
    __shared__ float s_rsum[kStRouterSlots][NT];
    __shared__ float s_pub[kBtMaxPublish];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kStConsumerWarps);

    unsigned char* ring = smem + p.off_ring;
    T* sdown_buf = reinterpret_cast<T*>(smem + p.off_sdown);
    T* xs = reinterpret_cast<T*>(smem + p.off_act);  // the normalised tokens as T [ntok][H]
    float* part = reinterpret_cast<float*>(smem + p.off_part);  // [npairs + ntok][hr_max]
    int* s_uniq_e = reinterpret_cast<int*>(smem + p.off_uniq_e);
    unsigned long long* s_uniq_m = reinterpret_cast<unsigned long long*>(smem + p.off_uniq_m);
    int* s_pair_e = reinterpret_cast<int*>(smem + p.off_pair_e);
    float* s_pair_w = reinterpret_cast<float*>(smem + p.off_pair_w);
    int4* desc = reinterpret_cast<int4*>(smem + p.off_desc);
    unsigned long long* s_emask = reinterpret_cast<unsigned long long*>(smem + p.off_emask);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_bar = full_bar + kStMaxStages;
    unsigned long long* topk_bar = empty_bar + kStMaxStages;  // one arrival per token: its routing is in shared memory
    unsigned long long* sdown_bar = topk_bar + 1;
    unsigned long long* route_bar = sdown_bar + 1;

    const T* x = static_cast<const T*>(p.x);
    const int R = p.nstages;
    const int PR = p.pr;
    const size_t rowH = (size_t)p.H;
    const size_t up_off = (size_t)PR * rowH;
    const int npairs = p.ntok * kBtPairStride;

    const int r0 = fdiv(p.E * cta, p.fd_ncta), r1 = fdiv(p.E * (cta + 1), p.fd_ncta);
    const int s0 = fdiv(p.Is * cta, p.fd_ncta), s1 = fdiv(p.Is * (cta + 1), p.fd_ncta);
    const int h0 = fdiv(p.H * cta, p.fd_ncta), h1 = fdiv(p.H * (cta + 1), p.fd_ncta);
    const int hr = h1 - h0;

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) {
        trace_stamp(p.ctl, 0);
        p.ctl->trace[22] = (unsigned long long)clock64();
    }
    if (tid == 0) cta_stamp(p.ctl, cta, 3);

    if (tid < 2 * kStMaxStages) mbar_init(&full_bar[tid], tid >= kStMaxStages ? kStConsumerWarps : 1);
    if (tid == 2 * kStMaxStages) mbar_init(topk_bar, (unsigned)p.ntok);
    if (tid == 2 * kStMaxStages + 1) mbar_init(sdown_bar, 1);
    if (tid == 2 * kStMaxStages + 2) mbar_init(route_bar, 1);
    if (tid == 0) {
        s_abort = 0;
        s_unique = 0;
        s_step = (p.comm.world > 1) ? comm_read_step(p.comm) : 0u;
    }
    for (int e = tid; e < p.E; e += kStThreads) s_emask[e] = 0ull;
    if (tid < 32) mbar_init_fence();
    __syncthreads();

    // =====================================================================================
    // Producer warp
    // =====================================================================================
    if (is_producer) {
        // nothing is issued on a workspace whose status is set (a CTA that leaves must have no copy in flight)
        int dirty = 0;
        if (lane == 0) {
            dirty = ld_volatile_s32(&p.ctl->status);
            if (dirty != 0) *(volatile int*)&s_abort = 1;
        }
        dirty = __shfl_sync(kFullMask, dirty, 0);
        if (dirty != 0) return;

        bool ok = true;
        int stage = 0, use = 0;
        auto acquire = [&]() -> bool {
            if (use > 0) ok = mbar_wait(&empty_bar[stage], (unsigned)(use - 1) & 1u, &s_abort);
            return ok;
        };
        auto advance = [&]() {
            if (++stage == R) { stage = 0; ++use; }
        };
        if (lane == 0) {
            for (int first = s0; first < s1 && ok; first += PR) {
                const int count = min(PR, s1 - first);
                const unsigned bytes = (unsigned)((size_t)count * rowH * sizeof(T));
                if (!acquire()) break;
                unsigned char* dst = ring + (size_t)stage * kStStageBytes;
                desc[stage] = make_int4(kChunkShared, 0, first, count);
                mbar_arrive_expect_tx(&full_bar[stage], 2 * bytes);
                bulk_copy_g2s(dst, static_cast<const T*>(p.sgate) + (size_t)first * rowH, bytes, &full_bar[stage]);
                bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.sup) + (size_t)first * rowH, bytes, &full_bar[stage]);
                advance();
            }
            if (p.Is > 0) {
                const unsigned bytes = (unsigned)((size_t)hr * p.Is * sizeof(T));
                mbar_arrive_expect_tx(sdown_bar, bytes);
                bulk_copy_g2s(sdown_buf, static_cast<const T*>(p.sdown) + (size_t)h0 * p.Is, bytes, sdown_bar);
            }
        }
        __syncwarp();

        // ---- the consumer warps route one token each; group the (token, slot) pairs by distinct local expert:
        //      the routing warps have marked, per expert, the pairs that chose it ----
        {
            int routed_ok = 0;
            if (lane == 0) routed_ok = mbar_wait(topk_bar, 0, &s_abort) ? 1 : 0;
            if (!__shfl_sync(kFullMask, routed_ok, 0)) return;  // copies in flight land on barriers the consumers wait on
        }
        if (cta == 0 && lane == 0) trace_stamp(p.ctl, 3);
        // distinct local experts in index order, each with the pairs that chose it: lane l scans experts 8 l .. 8 l + 7
        int n_unique = 0;
        {
            unsigned long long mm[kStTopkPerLane];
            int cnt = 0;
#pragma unroll
            for (int j = 0; j < kStTopkPerLane; ++j) {
                const int e = lane * kStTopkPerLane + j;
                mm[j] = (e < p.E) ? s_emask[e] : 0ull;
                cnt += (mm[j] != 0ull) ? 1 : 0;
            }
            int incl = cnt;
#pragma unroll
            for (int off = 1; off < 32; off <<= 1) {
                const int t = __shfl_up_sync(kFullMask, incl, off);
                if (lane >= off) incl += t;
            }
            n_unique = __shfl_sync(kFullMask, incl, 31);
            int pos = incl - cnt;
#pragma unroll
            for (int j = 0; j < kStTopkPerLane; ++j) {
                if (mm[j] != 0ull) {
                    s_uniq_e[pos] = lane * kStTopkPerLane + j;
                    s_uniq_m[pos] = mm[j];
                    ++pos;
                }
            }
        }
        __syncwarp();
        if (lane != 0) return;
        s_unique = n_unique;
        mbar_arrive(route_bar);  // releases the routing to the consumers
        if (cta == 0) trace_stamp(p.ctl, 4);

        // ---- routed gate/up chunks: PR consecutive channels of one expert, gate rows then up rows.  The first
        //      rounds are dealt statically, the rest through the counter (a CTA served faster takes more). ----
        {
            const int nchunks = n_unique * (int)p.fd_cpe.d;
            int static_rounds = fdiv(nchunks, p.fd_ncta);
            if (!p.deal_static) static_rounds = max(static_rounds - p.dyn_rounds, 0);
            const int dyn_base = static_rounds * ncta;
            int k = 0;
            int t_next = (k < static_rounds || p.deal_static) ? cta : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
#pragma unroll 1
            while (ok) {
                const int t = t_next;
                if (t >= nchunks) break;
                ++k;
                t_next = (k < static_rounds || p.deal_static) ? k * ncta + cta : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
                int u, ci;
                fdivmod(t, p.fd_cpe, u, ci);
                const int i0 = ci * PR;
                const int e = s_uniq_e[u] - p.expert_base;
                const unsigned bytes = (unsigned)((size_t)PR * rowH * sizeof(T));
                if (!acquire()) break;
                unsigned char* dst = ring + (size_t)stage * kStStageBytes;
                const size_t off = ((size_t)e * p.I + i0) * rowH;
                desc[stage] = make_int4(kChunkRouted, u, i0, PR);
                mbar_arrive_expect_tx(&full_bar[stage], 2 * bytes);
                bulk_copy_g2s(dst, static_cast<const T*>(p.egate) + off, bytes, &full_bar[stage]);
                bulk_copy_g2s(dst + up_off * sizeof(T), static_cast<const T*>(p.eup) + off, bytes, &full_bar[stage]);
                advance();
            }
        }
        if (cta == 0) trace_stamp(p.ctl, 16);
        // ---- the end mark: an empty chunk after which the consumers go to the grid barrier ----
        if (ok && acquire()) {
            desc[stage] = make_int4(kChunkEnd, 0, 0, 0);
            mbar_arrive(&full_bar[stage]);
            advance();
        }
        // ---- down rows of this CTA: one block of hr rows per distinct expert, `upc` blocks per stage ----
        const unsigned cbytes = (unsigned)((size_t)hr * p.I * sizeof(T));
        for (int j = 0; j < n_unique && ok; j += p.upc) {
            const int n = min(p.upc, n_unique - j);
            if (!acquire()) break;
            unsigned char* dst = ring + (size_t)stage * kStStageBytes;
            desc[stage] = make_int4(kChunkDown, j, n, 0);
            mbar_arrive_expect_tx(&full_bar[stage], cbytes * (unsigned)n);
            for (int q = 0; q < n; ++q) {
                const int e = s_uniq_e[j + q] - p.expert_base;
                bulk_copy_g2s(dst + (size_t)q * p.unit_bytes, static_cast<const T*>(p.edown) + ((size_t)e * p.H + h0) * p.I, cbytes, &full_bar[stage]);
            }
            advance();
        }
        if (cta == 0) trace_stamp(p.ctl, 18);
        if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingProducer);
        // Consumers wait on every barrier that was armed, and a wait only runs out long after any copy has
        // landed, so no copy into this CTA's shared memory is in flight when the CTA leaves.
        return;
    }

    // =====================================================================================
    // Consumer warps
    // =====================================================================================
    const int group = warp / kStGroupWarps;
    const int wi = warp % kStGroupWarps;

    int dirty = 0;
    unsigned epoch = 0;
    if (tid == 0) {
        dirty = ld_volatile_s32(&p.ctl->status);
        epoch = ld_volatile_u32(&p.ctl->epoch);
    }
    // the residual element this thread adds at the very end (one output element per thread): requested now
    float resid = 0.0f;
    {
        const int b = tid >> 4, j = tid & (kStMaxRows - 1);
        if (p.add_residual && tid < p.ntok * kStMaxRows && j < hr) resid = to_float<T>(x[(size_t)b * p.H + h0 + j]);
    }

    // ---- router rows of this CTA into registers, requested together with x and the norm weight ----
    const int npr = (int)p.fd_npr.d;
    const int rpieces = (r1 - r0) * npr;
    uint4 rp[kStRouterPieces];
#pragma unroll
    for (int i = 0; i < kStRouterPieces; ++i) {
        const int j = tid + i * kStConsumerThreads;
        rp[i] = make_uint4(0, 0, 0, 0);
        if (j < rpieces) rp[i] = ld_stream_u4(static_cast<const T*>(p.router_w) + (size_t)r0 * rowH + (size_t)j * 8);
    }

    // ---- RMSNorm of all tokens into shared memory (as T: the reference rounds the normalised input).
    //      Thread t owns the 16-byte piece t of every token; one block-wide exchange for all tokens. ----
    {
        const int k = tid * 8;
        const bool mine = k < p.H;
        uint4 xv[NT];
        uint4 wv = make_uint4(0, 0, 0, 0);
#pragma unroll
        for (int b = 0; b < NT; ++b) {
            xv[b] = make_uint4(0, 0, 0, 0);
            if (mine && b < p.ntok) xv[b] = *reinterpret_cast<const uint4*>(x + (size_t)b * p.H + k);
        }
        if (mine) wv = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + k);
        float ss[NT];
#pragma unroll
        for (int b = 0; b < NT; ++b) {
            float f[8];
            st_unpack<T>(xv[b], f);
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < 8; ++i) s = fmaf(f[i], f[i], s);
            ss[b] = s;
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int b = 0; b < NT; ++b) ss[b] += __shfl_xor_sync(kFullMask, ss[b], off);
        }
        if (lane < NT) {
            float mineval = ss[0];
#pragma unroll
            for (int b = 1; b < NT; ++b)
                if (lane == b) mineval = ss[b];
            s_red[warp][lane] = mineval;
        }
        named_barrier(1, kStConsumerThreads);
        float g[8];
        st_unpack<T>(wv, g);
#pragma unroll
        for (int b = 0; b < NT; ++b) {
            if (b < p.ntok) {
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < kStConsumerWarps; ++w) tot += s_red[w][b];
                const float rstd = 1.0f / sqrtf(tot / (float)p.H + p.eps);
                if (mine) {
                    float f[8];
                    st_unpack<T>(xv[b], f);
                    T o[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(f[i], rstd), g[i]));
                    *reinterpret_cast<uint4*>(xs + (size_t)b * p.H + k) = *reinterpret_cast<const uint4*>(o);
                }
            }
        }
        named_barrier(1, kStConsumerThreads);
    }
    if (tracer) trace_stamp(p.ctl, 1);

    // ---- router logits: a warp's 32 pieces lie in one row, so a warp sum gives the warp's share of that row ----
#pragma unroll
    for (int i = 0; i < kStRouterPieces; ++i) {
        const int j = tid + i * kStConsumerThreads;
        float acc[NT];
#pragma unroll
        for (int b = 0; b < NT; ++b) acc[b] = 0.0f;
        if (j < rpieces) {
            int row, piece;
            fdivmod(j, p.fd_npr, row, piece);
            float fw[8];
            st_unpack<T>(rp[i], fw);
#pragma unroll
            for (int b = 0; b < NT; ++b) {
                if (b < p.ntok) {
                    float fx[8];
                    st_unpack<T>(lds128(xs + (size_t)b * p.H + 8 * piece), fx);
#pragma unroll
                    for (int q = 0; q < 8; ++q) acc[b] = fmaf(fw[q], fx[q], acc[b]);
                }
            }
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
            for (int b = 0; b < NT; ++b) acc[b] += __shfl_xor_sync(kFullMask, acc[b], off);
        }
        if (lane < NT) {
            float v = acc[0];
#pragma unroll
            for (int b = 1; b < NT; ++b)
                if (lane == b) v = acc[b];
            s_rsum[i * kStConsumerWarps + warp][lane] = v;
        }
    }
    if (tid == 0) {
        s_epoch = epoch;
        if (dirty != 0) *(volatile int*)&s_abort = 1;
    }
    named_barrier(1, kStConsumerThreads);
    const int nrows = r1 - r0;
    const int npub = nrows * p.ntok;  // logits this CTA owes everybody: index v = b * rows + row
    if (tid < npub) {
        const int row = tid % nrows, b = tid / nrows;
        const int per_row = npr >> 5;  // 32-piece blocks per row
        float sum = 0.0f;
#pragma unroll 4
        for (int s = row * per_row; s < (row + 1) * per_row; ++s) sum += s_rsum[s][b];
        s_pub[tid] = sum;
    }
    named_barrier(1, kStConsumerThreads);
    const unsigned tag = s_epoch + 1u;
    if (*(volatile int*)&s_abort == 0) {
        // every logit into every mailbox; `box_share` neighbouring CTAs read the same one, which keeps the number
        // of stores in flight at that of a one-token launch and the readers of a line few
        const unsigned long long tagbits = (unsigned long long)tag << 32;
        const int nbox = (ncta + p.box_share - 1) / p.box_share;
        const int items = npub * nbox;
#pragma unroll 1
        for (int it = tid; it < items; it += kStConsumerThreads) {
            const int v = it / nbox, dest = it - v * nbox;
            const int row = v % nrows, b = v / nrows;
            const unsigned long long word = tagbits | (unsigned long long)__float_as_uint(s_pub[v]);
            st_relaxed_u64(p.mailbox + (size_t)dest * p.box_stride + b * p.E + r0 + row, word);
        }
    }
    if (tracer) trace_stamp(p.ctl, 2);
    if (tid == 0) cta_stamp(p.ctl, cta, 4);

    // ---- routing: warp b takes token b ----
    if (warp < p.ntok && *(volatile int*)&s_abort == 0) {
        RouteArgs ra;
        ra.box = p.mailbox + (size_t)(cta / p.box_share) * p.box_stride;
        ra.ctl = p.ctl;
        ra.indices = (cta == 0) ? p.indices : nullptr;
        ra.route_w = (cta == 0) ? p.route_w : nullptr;
        ra.emask = s_emask;
        ra.E = p.E;
        ra.K = p.K;
        ra.expert_base = p.expert_base;
        ra.local_experts = p.local_experts;
        if (route_token(ra, warp, tag, s_pair_e, s_pair_w, (volatile int*)&s_abort, lane)) {
            if (lane == 0) mbar_arrive(topk_bar);
            if (tid == 0) cta_stamp(p.ctl, cta, 6);
        }
    }

    bool ok = true;
    // chunk c is worked on by group (c + 2) % 3: the first chunk is the shared expert's, and groups 0 and 1 route
    int stage = 0, use = 0, owner = kStGroups - 1;
    bool routed = false;
    int4 d = make_int4(kChunkEnd, 0, 0, 0);
    const int nchH = p.H >> 3;
    auto wait_chunk = [&]() {
        if (ok) ok = mbar_wait(&full_bar[stage], (unsigned)use & 1u, &s_abort);
        if (ok) d = desc[stage];
        else d = make_int4(kChunkEnd, 0, 0, 0);
    };
    auto release_chunk = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == R) { stage = 0; ++use; }
        if (++owner == kStGroups) owner = 0;
    };

    // ---- gate/up chunks: shared expert first, then whatever the producer was dealt ----
    for (;;) {
        wait_chunk();
        if (d.x != kChunkShared && d.x != kChunkRouted) break;
        if (d.x == kChunkRouted && !routed) {
            ok = mbar_wait(route_bar, 0, &s_abort);
            routed = true;
            if (!ok) break;
            if (tracer) trace_stamp(p.ctl, 5);
        }
        if (owner == group) {
            const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kStStageBytes);
            const int count = d.w;
            const bool is_routed = (d.x == kChunkRouted);
            // bit q of the mask: routed: pair q (token q / K, result row q of act); shared: token q
            const unsigned long long mask = is_routed ? s_uniq_m[d.y] : ((1ull << p.ntok) - 1ull);
            float* obase = is_routed ? p.act : p.sact;
            const int olen = is_routed ? p.I : p.Is;
#pragma unroll 1
            for (int r = wi; r < count; r += kStGroupWarps) {
                const T* g = sbase + (size_t)r * rowH;
                const T* u = sbase + (size_t)(PR + r) * rowH;
                unsigned long long m = mask;
#pragma unroll 1
                while (m) {
                    const int q0 = __ffsll((long long)m) - 1;
                    m &= m - 1;
                    int q1 = -1;
                    if (m) {
                        q1 = __ffsll((long long)m) - 1;
                        m &= m - 1;
                    }
                    const int b0 = is_routed ? (q0 >> 3) : q0;
                    const T* x0 = xs + (size_t)b0 * rowH;
                    float* o0 = obase + (size_t)q0 * olen + d.z + r;
                    if (q1 < 0) {
                        const float4 s4 = pair_dot<T, 1>(g, u, x0, x0, nchH, lane);
                        if (lane == 0) *o0 = silu(s4.x) * s4.y;
                    } else {
                        const int b1 = is_routed ? (q1 >> 3) : q1;
                        const float4 s4 = pair_dot<T, 2>(g, u, x0, xs + (size_t)b1 * rowH, nchH, lane);
                        if (lane == 0) {
                            *o0 = silu(s4.x) * s4.y;
                            *(obase + (size_t)q1 * olen + d.z + r) = silu(s4.z) * s4.w;
                        }
                    }
                }
            }
        }
        release_chunk();
    }
    if (ok && d.x != kChunkEnd) ok = false;  // cannot happen: the gate/up stream ends with the end mark
    if (ok) release_chunk();                 // the end mark's stage goes back to the producer
    if (ok && !routed) ok = mbar_wait(route_bar, 0, &s_abort);
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);

    // ---- the grid barrier: every CTA's activations are in the scratch buffers ----
    if (tracer) trace_stamp(p.ctl, 6);
    named_barrier(1, kStConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 0);
    if (tid == 0) {
        bool fine = ok && (*(volatile int*)&s_abort == 0);
        if (fine) {
            const unsigned target = barrier_arrive(p.ctl, ncta, 0);
            fine = barrier_wait(p.ctl, target, kStatusMoeBarrier2);
            if (fine) barrier_finish(p.ctl, ncta);
        }
        if (!fine) *(volatile int*)&s_abort = 1;
        s_flag = fine ? 1 : 0;
    }
    named_barrier(1, kStConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 7);
    if (tid == 0) cta_stamp(p.ctl, cta, 1);
    if (!s_flag) return;  // every consumer warp leaves; the producer sees the abort flag in its waits
    const int n_unique = s_unique;

    float a[2][2][8];
    const int nchI = p.I >> 3, nchIs = p.Is >> 3;
    // ---- the shared expert's down rows, by groups 1 and 2: warp = (token pair, half of the rows).  Group 0
    //      starts on the routed chunks at once; the ring is deep enough to cover the others' detour. ----
    if (p.Is > 0 && group >= 1) {
        const int b0 = 2 * wi;
        if (b0 < p.ntok) {
            ok = mbar_wait(sdown_bar, 0, &s_abort);
            if (ok) {
                const int lo = (hr * (group - 1)) / 2, hi = (hr * group) / 2;
                const unsigned long long m = (b0 + 1 < p.ntok) ? 3ull : 1ull;
                if (lo < hi)
                    down_block_rows<T>(sdown_buf, lo, hi, nchIs, m, p.sact + (size_t)b0 * p.Is, p.Is, part + (size_t)(npairs + b0) * p.hr_max, p.hr_max,
                                       false, a, lane);
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 8);

    // ---- the routed experts' down rows: chunk = up to `upc` blocks of hr rows; the owning group's four warps
    //      cut the chunk's rows into four runs.  What a warp will need of the activations is known before
    //      the chunk arrives, so the first vectors are requested before the wait. ----
#pragma unroll 1
    for (int done = 0; done < n_unique && ok;) {
        const int n = min(p.upc, n_unique - done);
        const bool mine = (owner == group);
        int f0 = 0, f1 = 0, q_first = 0;
        bool pre = false;
        if (mine) {
            const int total = n * hr;
            f0 = (total * wi) / kStGroupWarps;
            f1 = (total * (wi + 1)) / kStGroupWarps;
            if (f0 < f1) {
                q_first = f0 / hr;
                unsigned long long m = s_uniq_m[done + q_first];
                const int q0 = __ffsll((long long)m) - 1;
                m &= m - 1;
                if (m) load_acts<2>(p.act + (size_t)q0 * p.I, p.act + (size_t)(__ffsll((long long)m) - 1) * p.I, nchI, lane, a);
                else load_acts<1>(p.act + (size_t)q0 * p.I, p.act, nchI, lane, a);
                pre = true;
            }
        }
        wait_chunk();
        if (!ok) break;
        if (d.x != kChunkDown || d.y != done || d.z != n) { ok = false; break; }  // cannot happen
        if (mine && f0 < f1) {
            const unsigned char* sbase = ring + (size_t)stage * kStStageBytes;
#pragma unroll 1
            for (int q = q_first; q < n; ++q) {
                const int base = q * hr;
                const int lo = max(f0, base) - base, hi = min(f1, base + hr) - base;
                if (lo >= hi) break;
                down_block_rows<T>(reinterpret_cast<const T*>(sbase + (size_t)q * p.unit_bytes), lo, hi, nchI, s_uniq_m[done + q], p.act, p.I, part,
                                   p.hr_max, pre && q == q_first, a, lane);
            }
        }
        release_chunk();
        done += n;
    }
    if (tracer) trace_stamp(p.ctl, 14);
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    named_barrier(1, kStConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 2);
    if (*(volatile int*)&s_abort != 0 || !ok) return;

    // ---- combine in slot order, add the residual, round once: one output element per thread ----
    T* out = static_cast<T*>(p.out);
    const bool exchange = p.comm.world > 1;
    const unsigned step = s_step;
    if (tid < p.ntok * kStMaxRows) {
        const int b = tid >> 4, j = tid & (kStMaxRows - 1);
        if (j < hr) {
            float v = 0.0f;
#pragma unroll 4
            for (int k = 0; k < p.K; ++k) {
                const int pair = b * kBtPairStride + k;
                const int e = s_pair_e[pair];
                if (e >= p.expert_base && e < p.expert_base + p.local_experts) v = fmaf(s_pair_w[pair], part[pair * p.hr_max + j], v);
            }
            if (p.Is > 0) v += part[(npairs + b) * p.hr_max + j];
            const size_t o = (size_t)b * p.H + h0 + j;
            if (exchange) {
                comm_put(p.comm, step, o, v);
                if (comm_get_sum(p.comm, p.ctl, step, o, &v)) out[o] = from_float<T>(v + resid);
            } else if (p.partial_out) {
                p.partial_out[o] = v;
            } else {
                out[o] = from_float<T>(v + resid);
            }
        }
    }
    if (exchange && cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);
    if (tracer) {
        trace_stamp(p.ctl, 9);
        p.ctl->trace[23] = (unsigned long long)clock64();
    }
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------

// Launches the batch kernel, eight tokens per launch, when the call suits it (any token count; the dispatcher sends it calls of two or more; 2-byte
// dtype, aligned shapes) and sets *handled; otherwise leaves *handled false (no error).
int moe_decode_batch_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                            bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    if (a->batch < 1) return MK36_OK;
    const int H = a->hidden, E = a->experts, K = a->top_k, I = a->intermediate, Is = a->shared_intermediate;
    int tb = kBtMaxTokens;
    if (K <= 0 || K > kBtPairStride || I <= 0 || Is < 0 || E <= 0 || E > 32 * kStTopkPerLane) return MK36_OK;
    while (tb > 1 && (tb * kBtPairStride > kStMaxPairs || tb * E > kTagSlots)) --tb;
    if (a->batch < tb) tb = a->batch;
    if (H % 256 != 0 || I % 32 != 0 || Is % 32 != 0) return MK36_OK;  // a warp's 32 router pieces lie in one row
    if (I > 512 || Is > 512) return MK36_OK;  // the down phase keeps an activation vector in registers, 16 values per lane
    int pr = kStStageBytes / (H * 2) / 2;  // (gate, up) pairs per stage
    if (pr > 8) pr = 8;
    if (pr < 1 || I % pr != 0) return MK36_OK;
    const void* ptrs[] = {a->x, a->norm_weight, a->router_weight, a->expert_gate, a->expert_up, a->expert_down,
                          a->shared_gate, a->shared_up, a->shared_down};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const int ncta = dev->sm_count;
    if (H < ncta || (long long)H * ncta >= (1ll << 31) || (long long)E * ncta >= (1ll << 31) || (long long)Is * ncta >= (1ll << 31)) return MK36_OK;
    const int hr_max = (H + ncta - 1) / ncta;
    if (hr_max > kStMaxRows) return MK36_OK;
    const int rows_max = (E + ncta - 1) / ncta + 1;
    if ((long long)rows_max * (H / 8) > (long long)kStRouterPieces * kStConsumerThreads) return MK36_OK;
    if (rows_max * tb > kBtMaxPublish) return MK36_OK;
    if (H > 8 * kStConsumerThreads) return MK36_OK;  // one 16-byte piece of each token per consumer thread
    const size_t unit_bytes = (size_t)hr_max * I * 2;
    if (unit_bytes > (size_t)kStStageBytes || (size_t)hr_max * Is * 2 > 65536) return MK36_OK;
    if ((long long)tb * K * (I / pr) * 2 >= (1ll << 31)) return MK36_OK;

    MoeStreamParams p;
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
    const int pairs = tb * kBtPairStride;
    p.off_bars = take((2 * kStMaxStages + 3) * 8, 16);
    p.off_desc = take(kStMaxStages * 16, 16);
    p.off_uniq_e = take(kStMaxPairs * 4, 16);
    p.off_uniq_m = take(kStMaxPairs * 8, 16);
    p.off_pair_e = take(kStMaxPairs * 4, 16);
    p.off_pair_w = take(kStMaxPairs * 4, 16);
    p.off_emask = take((size_t)E * 8, 16);
    p.off_part = take((size_t)(pairs + tb) * hr_max * 4, 16);
    p.off_sdown = take((size_t)hr_max * Is * 2, 128);
    p.off_act = take((size_t)tb * H * 2, 128);
    p.off_ring = take(0, 128);
    p.off_ded = 0;
    const long long room = (long long)dev->max_smem_optin - (long long)off - 2048;  // 2048: the kernel's static shared memory
    int nstages = options().moe_stages > 0 ? options().moe_stages : 5;
    if (nstages > kStMaxStages) nstages = kStMaxStages;
    while (nstages > 2 && (long long)nstages * kStStageBytes > room) --nstages;
    if ((long long)nstages * kStStageBytes > room || nstages < 2) return MK36_OK;
    const size_t smem_bytes = (size_t)p.off_ring + (size_t)nstages * kStStageBytes;

    const size_t scratch = align_up((size_t)tb * E * 4, 256) + align_up((size_t)pairs * I * 4, 256) + align_up((size_t)tb * (Is > 0 ? Is : 1) * 4, 256);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + scratch)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, kControlBytes + scratch);
    // the mailboxes live at a fixed offset that nothing else writes; a smaller workspace takes the ring kernel
    if (ncta > kMailboxMaxCtas || workspace_bytes < kTaggedEnd || kControlBytes + scratch > kMailboxOffset) return MK36_OK;

    p.norm_w = a->norm_weight;
    p.router_w = a->router_weight;
    p.egate = a->expert_gate;
    p.eup = a->expert_up;
    p.edown = a->expert_down;
    p.sgate = a->shared_gate;
    p.sup = a->shared_up;
    p.sdown = a->shared_down;
    p.ctl = static_cast<Control*>(workspace);
    p.mailbox = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(workspace) + kMailboxOffset);
    unsigned char* sc = static_cast<unsigned char*>(workspace) + kControlBytes + align_up((size_t)tb * E * 4, 256);
    p.act = reinterpret_cast<float*>(sc);
    sc += align_up((size_t)pairs * I * 4, 256);
    p.sact = reinterpret_cast<float*>(sc);
    p.H = H; p.E = E; p.K = K; p.I = I; p.Is = Is;
    p.expert_base = a->expert_base;
    p.local_experts = a->local_experts;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    p.nstages = nstages;
    p.nded = 0;
    p.pr = pr;
    p.hr_max = hr_max;
    p.unit_bytes = (int)unit_bytes;
    p.upc = (int)(kStStageBytes / unit_bytes);
    p.deal_static = options().moe_static ? 1 : 0;
    p.dyn_rounds = options().moe_dyn_rounds > 0 ? options().moe_dyn_rounds : 2;
    p.fd_ncta = make_fastdiv(ncta);
    p.fd_cpe = make_fastdiv(I / pr);
    p.fd_K = make_fastdiv(K);
    p.fd_qi = make_fastdiv(I / 4);
    p.fd_qis = make_fastdiv(Is > 0 ? Is / 4 : 1);
    p.fd_npr = make_fastdiv(H / 8);

    const void* kernel = (a->dtype == MK36_BF16) ? (const void*)moe_decode_batch_kernel<__nv_bfloat16> : (const void*)moe_decode_batch_kernel<__half>;
    {
        const int rc_smem = ensure_dynamic_smem(kernel, smem_bytes);
        if (rc_smem != MK36_OK) return rc_smem;
    }
    const size_t es = 2;
    for (int b0 = 0; b0 < a->batch; b0 += tb) {
        p.ntok = (a->batch - b0 < tb) ? (a->batch - b0) : tb;
        p.box_share = p.ntok;
        p.box_stride = (p.ntok * E + 511) / 512 * 512;
        p.x = static_cast<const unsigned char*>(a->x) + (size_t)b0 * H * es;
        p.out = a->out ? static_cast<unsigned char*>(a->out) + (size_t)b0 * H * es : nullptr;
        p.partial_out = a->partial_out ? a->partial_out + (size_t)b0 * H : nullptr;
        p.indices = a->indices ? reinterpret_cast<long long*>(a->indices) + (size_t)b0 * K : nullptr;
        p.route_w = a->route_weights ? a->route_weights + (size_t)b0 * K : nullptr;
        void* params[] = {&p};
        const int rc = launch_cooperative(kernel, dim3(ncta), dim3(kStThreads), smem_bytes, stream, params, "moe_decode(batch)");
        if (rc != MK36_OK) return rc;
    }
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
