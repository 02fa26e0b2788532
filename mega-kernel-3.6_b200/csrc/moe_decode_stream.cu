// MoE decode for launches of one token (two if asked to) on sm_100a (2-byte dtypes, aligned shapes): the
// latency-critical case, where the step moves ~400 KB per SM and its time is a chain of dependent
// latencies rather than a bandwidth problem.  Same results as the general kernel in moe_decode.cu
// (reference semantics: mega_kernel_qwen36/reference.py:16-62); replaces the seven grid-synchronised
// phases of csrc/persistent_moe_decode.cu:477-581 with one launch, one grid barrier and one weight
// stream that does not stop once the routing is known.
//
//   consumers (12 warps)                                 producer warp
//   ------------------------------------------------     ---------------------------------------------
//   x, norm weight and this CTA's router rows are        shared-expert gate/up rows and this CTA's rows
//   loaded together (one memory round trip); RMSNorm;     of shared_down are requested at entry
//   router dot products; every logit is pushed into
//   every CTA's own mailbox as a tagged 64-bit word -->  all lanes poll the CTA's mailbox: a word is its own
//   shared-expert (gate, up) pairs from the ring          ready flag, so there is no grid barrier, no second
//                                                         round trip and no line that many CTAs poll; top-k
//   routed (gate, up) pairs from the ring  <------------  and soft-max in registers; routed gate/up chunks
//   silu(g) * u -> global scratch                         are dealt to the CTAs through a work counter (a
//   grid barrier (the only one)                           CTA that is served faster takes more), and the
//   activations -> shared memory                          down rows of this CTA are requested right behind
//   down rows (resident or in flight) -> partial sums     the last gate/up chunk, into slots of their own
//   combine in slot order, residual, store / exchange     and, when those are full, into freed ring stages
//
// The ring is one in-order sequence of 32 KB stages.  Chunk c lives in stage c % depth and is worked
// on by consumer group c % 3, but every consumer warp waits for every chunk and releases it: all
// warps see every barrier phase exactly once, in order (a warp that skipped phases could mistake an
// older phase for the one it waits for), and all warps learn from the chunk's descriptor when the
// gate/up stream of this CTA has ended.  The descriptor (what the stage holds) is written by the
// producer before it arms the stage, because with dealt work the consumers cannot compute it.
//
// Contractions are plain FMAs with warp-shuffle reductions: at one or two token columns a 16 x 8
// tensor-core tile would be almost all padding, and the warp-level mma.sync of this part is slow
// enough that unpack + FMA costs no more issue cycles.
#include "mk36_moe_stream.cuh"

namespace mk36 {

template <typename T, int NT>
__global__ void __launch_bounds__(kStThreads, 1) moe_decode_stream_kernel(const MoeStreamParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_unique;
    __shared__ int s_abort;
    __shared__ unsigned s_step;
    __shared__ unsigned s_epoch;
    __shared__ float s_red[kStConsumerWarps];
    __shared__ float s_rsum[kStRouterSlots][NT];
    __shared__ float s_pub[kStMaxPublish];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kStConsumerWarps);

    unsigned char* ring = smem + p.off_ring;
    unsigned char* ded = smem + p.off_ded;
    T* sdown_buf = reinterpret_cast<T*>(smem + p.off_sdown);
    T* xs = reinterpret_cast<T*>(smem + p.off_act);       // until the grid barrier: tokens as T [ntok][H]
    float* actf = reinterpret_cast<float*>(smem + p.off_act);  // afterwards: activations, fp32
    float* part = reinterpret_cast<float*>(smem + p.off_part);  // [npairs + ntok][hr_max]
    int* s_uniq_e = reinterpret_cast<int*>(smem + p.off_uniq_e);
    unsigned long long* s_uniq_m = reinterpret_cast<unsigned long long*>(smem + p.off_uniq_m);
    int* s_pair_e = reinterpret_cast<int*>(smem + p.off_pair_e);
    float* s_pair_w = reinterpret_cast<float*>(smem + p.off_pair_w);
    int4* desc = reinterpret_cast<int4*>(smem + p.off_desc);
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_bar = full_bar + kStMaxStages;
    unsigned long long* ded_bar = empty_bar + kStMaxStages;
    unsigned long long* sdown_bar = ded_bar + kStMaxDed;
    unsigned long long* route_bar = sdown_bar + 1;

    const T* x = static_cast<const T*>(p.x);
    const int R = p.nstages;
    const int PR = p.pr;
    const size_t rowH = (size_t)p.H;
    const size_t up_off = (size_t)PR * rowH;  // element offset of the up rows inside a stage
    const int npairs = p.ntok * p.K;

    // ---- static partition: router rows, shared-expert channels and output rows of this CTA ----
    const int r0 = fdiv(p.E * cta, p.fd_ncta), r1 = fdiv(p.E * (cta + 1), p.fd_ncta);
    const int s0 = fdiv(p.Is * cta, p.fd_ncta), s1 = fdiv(p.Is * (cta + 1), p.fd_ncta);
    const int h0 = fdiv(p.H * cta, p.fd_ncta), h1 = fdiv(p.H * (cta + 1), p.fd_ncta);
    const int hr = h1 - h0;

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) {
        trace_stamp(p.ctl, 0);
        p.ctl->trace[22] = (unsigned long long)clock64();  // with slot 23: SM cycles per nanosecond of this launch
    }
    if (tid == 0) cta_stamp(p.ctl, cta, 3);

    // one barrier per thread: full[0..5], empty[0..5], ded[0..15], sdown, route are contiguous
    if (tid < 2 * kStMaxStages + kStMaxDed + 2) {
        const bool is_empty = tid >= kStMaxStages && tid < 2 * kStMaxStages;
        mbar_init(&full_bar[tid], is_empty ? kStConsumerWarps : 1);
    }
    if (tid == 0) {
        s_abort = 0;
        s_unique = 0;
        s_step = (p.comm.world > 1) ? comm_read_step(p.comm) : 0u;
    }
    if (tid < 32) mbar_init_fence();
    __syncthreads();

    // =====================================================================================
    // Producer warp
    // =====================================================================================
    if (is_producer) {
        // status word and epoch share a line of the control block.  The producer waits for them
        // before it issues anything: on a workspace whose status is set nothing may run, and a CTA
        // that leaves must have no copy in flight into its shared memory.
        unsigned epoch = 0;
        int dirty = 0;
        if (lane == 0) {
            dirty = ld_volatile_s32(&p.ctl->status);
            epoch = ld_volatile_u32(&p.ctl->epoch);
            if (dirty != 0) *(volatile int*)&s_abort = 1;
        }
        dirty = __shfl_sync(kFullMask, dirty, 0);
        epoch = __shfl_sync(kFullMask, epoch, 0);
        if (dirty != 0) return;
        const unsigned tag = epoch + 1u;

        bool ok = true;
        int c = 0, stage = 0, use = 0;  // next chunk of the ring: its stage and how often the stage was used before
        // stage for the next chunk, once the consumers have released its previous contents
        auto acquire = [&]() -> bool {
            if (use > 0) ok = mbar_wait(&empty_bar[stage], (unsigned)(use - 1) & 1u, &s_abort);
            return ok;
        };
        auto advance = [&]() {
            ++c;
            if (++stage == R) { stage = 0; ++use; }
        };
        if (lane == 0) {
            // shared expert: gate and up rows s0..s1 (contiguous in memory), and this CTA's rows of shared_down
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

        // ---- every CTA's logits: poll this CTA's mailbox until all words carry this kernel's tag.  Logits
        //      become order-preserving unsigned keys (larger logit = larger key); 0 = no logit / already taken ----
        unsigned key[NT][kStTopkPerLane];
        {
            const unsigned long long* box = p.mailbox + (size_t)cta * p.box_stride;
            const unsigned long long t0 = global_timer_ns();
            unsigned spins = 0;
            unsigned have = 0u;  // bit b * 8 + j: that word has arrived (it is not asked for again)
            for (;;) {
                bool ready = true;
#pragma unroll
                for (int b = 0; b < NT; ++b) {
#pragma unroll
                    for (int j = 0; j < kStTopkPerLane; ++j) {
                        const int e = lane + 32 * j;
                        const unsigned bit = 1u << (b * kStTopkPerLane + j);
                        if (b < p.ntok && e < p.E) {
                            if (!(have & bit)) {
                                const unsigned long long w = ld_relaxed_u64(box + b * p.E + e);
                                if ((unsigned)(w >> 32) == tag) {
                                    have |= bit;
                                    const unsigned bits = (unsigned)w;
                                    key[b][j] = topk_key(bits);
                                } else {
                                    ready = false;
                                }
                            }
                        } else {
                            key[b][j] = 0u;
                        }
                    }
                }
                if (__all_sync(kFullMask, ready)) break;
                if ((++spins & 15u) == 0u) {
                    bool give_up = false;
                    if (lane == 0) {
                        if (*(volatile int*)&s_abort != 0) give_up = true;
                        else if (global_timer_ns() - t0 > kWaitLimitNs) {
                            atomicCAS(&p.ctl->status, 0, kStatusMoeLogits);
                            *(volatile int*)&s_abort = 1;
                            give_up = true;
                        }
                    }
                    if (__shfl_sync(kFullMask, give_up ? 1 : 0, 0)) { ok = false; break; }
                }
            }
            if (!ok) return;  // nothing is in flight except copies whose barriers the consumers wait on
            if (cta == 0 && lane == 0) trace_stamp(p.ctl, 3);
        }

        // ---- top-k (descending logit, lowest index on ties) and soft-max over the k survivors, per token.
        //      A round is one warp-wide maximum of the lanes' best keys; the lane that holds it records the
        //      selection itself, so nothing else crosses the warp unless several lanes tie. ----
#pragma unroll 1
        for (int b = 0; b < p.ntok; ++b) {
            unsigned k8[kStTopkPerLane];
#pragma unroll
            for (int j = 0; j < kStTopkPerLane; ++j) k8[j] = (NT > 1 && b == 1) ? key[NT - 1][j] : key[0][j];
            topk_select(k8, p.K, lane, [&](int r, int e, float logit) {
                s_pair_e[b * p.K + r] = e;
                s_pair_w[b * p.K + r] = logit;
            });
            __syncwarp();
            const float first = s_pair_w[b * p.K];
            const float ev = (lane < p.K) ? expf(s_pair_w[b * p.K + lane] - first) : 0.0f;
            const float denom = warp_sum(ev);
            if (lane < p.K) {
                const float w = ev / denom;
                s_pair_w[b * p.K + lane] = w;
                if (cta == 0) {
                    if (p.indices) p.indices[(size_t)b * p.K + lane] = (long long)s_pair_e[b * p.K + lane];
                    if (p.route_w) p.route_w[(size_t)b * p.K + lane] = w;
                }
            }
        }
        __syncwarp();
        // group the (token, slot) pairs by distinct local expert: the leader of a group is its lowest pair
        // index; leaders are listed in pair order
        int n_unique = 0;
        if (npairs <= 32) {
            const int e = (lane < npairs) ? s_pair_e[lane] : -1 - lane;
            const bool local = lane < npairs && e >= p.expert_base && e < p.expert_base + p.local_experts;
            const unsigned same = __match_any_sync(kFullMask, e);
            const bool leader = local && (__ffs((int)same) - 1) == lane;
            const unsigned vote = __ballot_sync(kFullMask, leader);
            if (leader) {
                const int pos = __popc(vote & ((1u << lane) - 1u));
                s_uniq_e[pos] = e;
                s_uniq_m[pos] = (unsigned long long)same;
            }
            n_unique = __popc(vote);
        } else {
#pragma unroll 1
            for (int base = 0; base < npairs; base += 32) {
                const int t = base + lane;
                unsigned long long m = 0ull;
                bool leader = false;
                if (t < npairs) {
                    const int e = s_pair_e[t];
                    if (e >= p.expert_base && e < p.expert_base + p.local_experts) {
#pragma unroll 1
                        for (int q = 0; q < npairs; ++q)
                            if (s_pair_e[q] == e) m |= 1ull << q;
                        leader = (__ffsll((long long)m) - 1) == t;
                    }
                }
                const unsigned vote = __ballot_sync(kFullMask, leader);
                if (leader) {
                    const int pos = n_unique + __popc(vote & ((1u << lane) - 1u));
                    s_uniq_e[pos] = s_pair_e[t];
                    s_uniq_m[pos] = m;
                }
                n_unique += __popc(vote);
            }
        }
        __syncwarp();
        if (lane != 0) return;
        s_unique = n_unique;
        mbar_arrive(route_bar);  // releases the routing to the consumers
        if (cta == 0) trace_stamp(p.ctl, 4);

        // ---- routed gate/up chunks: PR consecutive channels of one expert, gate rows then up rows ----
        {
            const int nchunks = n_unique * (int)p.fd_cpe.d;
            // the first rounds are dealt statically (no counter traffic while everybody starts), the rest through
            // the counter, so that CTAs whose memory is served faster end up with more chunks
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
                // the next ticket is in flight while this chunk waits for its stage
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
                if (cta == 0 && k == 1) trace_stamp(p.ctl, 15);
                advance();
            }
        }
        if (cta == 0) trace_stamp(p.ctl, 16);

        // ---- down rows of this CTA, one block of hr rows per distinct expert: right behind the gate/up stream ----
        const unsigned cbytes = (unsigned)((size_t)hr * p.I * sizeof(T));
        const int nd = min(p.nded, n_unique);
        for (int j = 0; j < nd && ok; ++j) {
            const int e = s_uniq_e[j] - p.expert_base;
            mbar_arrive_expect_tx(&ded_bar[j], cbytes);
            bulk_copy_g2s(ded + (size_t)j * p.unit_bytes, static_cast<const T*>(p.edown) + ((size_t)e * p.H + h0) * p.I, cbytes, &ded_bar[j]);
        }
        if (cta == 0) trace_stamp(p.ctl, 17);
        for (int j = nd; j < n_unique && ok; j += p.upc) {
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
        if (nd == n_unique && ok && acquire()) {
            // no down chunk goes through the ring: an empty chunk tells the consumers that the gate/up stream has ended
            desc[stage] = make_int4(kChunkEnd, 0, 0, 0);
            mbar_arrive(&full_bar[stage]);
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

    // status and epoch: requested now, looked at when the logits are ready to be published
    int dirty = 0;
    unsigned epoch = 0;
    if (tid == 0) {
        dirty = ld_volatile_s32(&p.ctl->status);
        epoch = ld_volatile_u32(&p.ctl->epoch);
    }
    // the residual element this thread will add at the very end (one output element per thread): requested now
    float resid = 0.0f;
    {
        const int b = tid >> 4, j = tid & (kStMaxRows - 1);
        if (p.add_residual && tid < p.ntok * kStMaxRows && j < hr) resid = to_float<T>(x[(size_t)b * p.H + h0 + j]);
    }

    // ---- router rows of this CTA straight into registers (r0..r1 are contiguous in memory), requested
    //      together with x and the norm weight so that the front costs one memory round trip ----
    const int npr = (int)p.fd_npr.d;  // 16-byte pieces per row of length hidden
    const int rpieces = (r1 - r0) * npr;
    uint4 rp[kStRouterPieces];
#pragma unroll
    for (int i = 0; i < kStRouterPieces; ++i) {
        const int j = tid + i * kStConsumerThreads;
        rp[i] = make_uint4(0, 0, 0, 0);
        if (j < rpieces) rp[i] = ld_stream_u4(static_cast<const T*>(p.router_w) + (size_t)r0 * rowH + (size_t)j * 8);
    }

    // ---- RMSNorm of the tokens into shared memory (as T: the reference rounds the normalised input) ----
#pragma unroll 1
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
        st_unpack<T>(xv, f);
        st_unpack<T>(wv, g);
        float ss = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
        ss = warp_sum(ss);
        if (lane == 0) s_red[warp] = ss;
        named_barrier(1, kStConsumerThreads);
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kStConsumerWarps; ++w) tot += s_red[w];
        const float rstd = 1.0f / sqrtf(tot / (float)p.H + p.eps);
        if (mine) {
            T o[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(f[i], rstd), g[i]));
            *reinterpret_cast<uint4*>(xs + (size_t)b * p.H + k) = *reinterpret_cast<const uint4*>(o);
        }
        named_barrier(1, kStConsumerThreads);
    }
    if (tracer) trace_stamp(p.ctl, 1);

    // ---- router logits: a warp's 32 pieces lie in one row (hidden / 8 is a multiple of 32), so a warp sum
    //      gives the warp's share of that row; the shares are added in a fixed order ----
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
        for (int b = 0; b < NT; ++b) acc[b] = warp_sum(acc[b]);
        // piece j sits in 32-piece block j / 32 = warp + 12 i: the blocks of a row are consecutive slots
        if (lane == 0) {
#pragma unroll
            for (int b = 0; b < NT; ++b) s_rsum[i * kStConsumerWarps + warp][b] = acc[b];
        }
    }
    if (tid == 0) {
        s_epoch = epoch;
        if (dirty != 0) *(volatile int*)&s_abort = 1;
    }
    named_barrier(1, kStConsumerThreads);
    const int npub = (r1 - r0) * p.ntok;  // logits this CTA owes everybody: index v = b * rows + row
    if (tid < npub) {
        const int row = tid % (r1 - r0), b = tid / (r1 - r0);
        const int per_row = npr >> 5;  // 32-piece blocks per row
        float sum = 0.0f;
#pragma unroll 4
        for (int s = row * per_row; s < (row + 1) * per_row; ++s) sum += s_rsum[s][NT > 1 ? b : 0];
        s_pub[tid] = sum;
    }
    named_barrier(1, kStConsumerThreads);
    if (*(volatile int*)&s_abort == 0) {
        // every logit into every CTA's mailbox: thread t serves the receivers t, t + 384, ...
        const unsigned long long tagbits = (unsigned long long)(s_epoch + 1u) << 32;
#pragma unroll 1
        for (int v = 0; v < npub; ++v) {
            const int row = v % (r1 - r0), b = v / (r1 - r0);
            const unsigned long long word = tagbits | (unsigned long long)__float_as_uint(s_pub[v]);
            for (int dest = tid; dest < ncta; dest += kStConsumerThreads)
                st_relaxed_u64(p.mailbox + (size_t)dest * p.box_stride + b * p.E + r0 + row, word);
        }
    }
    if (tracer) trace_stamp(p.ctl, 2);
    if (tid == 0) cta_stamp(p.ctl, cta, 4);

    bool ok = true;
    int c = 0, stage = 0, use = 0, owner = 0;  // chunk counter, its stage, earlier uses of the stage, c % groups
    bool routed = false;
    int4 d = make_int4(kChunkEnd, 0, 0, 0);
    const int nchH = p.H >> 3;
    auto next_chunk = [&]() {
        ++c;
        if (++stage == R) { stage = 0; ++use; }
        if (++owner == kStGroups) owner = 0;
    };
    auto wait_chunk = [&]() {
        if (ok) ok = mbar_wait(&full_bar[stage], (unsigned)use & 1u, &s_abort);
        if (ok) d = desc[stage];
        else d = make_int4(kChunkEnd, 0, 0, 0);
    };
    auto release_chunk = [&]() {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        next_chunk();
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
#pragma unroll 1
            for (int r = wi; r < count; r += kStGroupWarps) {
                const T* g = sbase + (size_t)r * rowH;
                const T* u = sbase + (size_t)(PR + r) * rowH;
                // the one or two token vectors this pair meets, and where the results go
                const T* x0 = xs;
                const T* x1 = xs + rowH;
                float* o0 = p.sact + d.z + r;
                float* o1 = p.sact + (size_t)p.Is + d.z + r;
                bool two = (NT > 1 && p.ntok > 1);
                if (d.x == kChunkRouted) {
                    const unsigned long long m = s_uniq_m[d.y];
                    const int p0 = __ffsll((long long)m) - 1;
                    const unsigned long long m1 = m & (m - 1);
                    const int p1 = m1 ? __ffsll((long long)m1) - 1 : p0;
                    x0 = xs + (size_t)fdiv(p0, p.fd_K) * rowH;
                    x1 = xs + (size_t)fdiv(p1, p.fd_K) * rowH;
                    o0 = p.act + (size_t)p0 * p.I + d.z + r;
                    o1 = p.act + (size_t)p1 * p.I + d.z + r;
                    two = (NT > 1 && m1 != 0ull);
                }
                if (!two) {
                    const float4 s4 = pair_dot<T, 1>(g, u, x0, x0, nchH, lane);
                    if (lane == 0) *o0 = silu(s4.x) * s4.y;
                } else {
                    const float4 s4 = pair_dot<T, (NT > 1 ? 2 : 1)>(g, u, x0, x1, nchH, lane);
                    if (lane == 0) {
                        *o0 = silu(s4.x) * s4.y;
                        *o1 = silu(s4.z) * s4.w;
                    }
                }
            }
        }
        release_chunk();
    }
    if (ok && !routed) ok = mbar_wait(route_bar, 0, &s_abort);
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);

    // ---- the grid barrier: every CTA's activations are in the scratch buffers ----
    if (tracer) trace_stamp(p.ctl, 6);
    named_barrier(1, kStConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 0);
    if (tid == 0) {
        bool fine = (*(volatile int*)&s_abort == 0);
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

    // ---- activations of the local pairs and of the shared expert into shared memory (the token region is
    //      reused).  All loads of a thread are issued before the first store. ----
    const size_t shared_base = (size_t)npairs * p.I;
    {
        const int q_i = p.I >> 2, q_is = p.Is >> 2;
        const int routed_items = npairs * q_i;
        const int items = routed_items + p.ntok * q_is;
#pragma unroll 1
        for (int base = 0; base < items; base += 4 * kStConsumerThreads) {
            float4 val[4];
            int dst[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                const int it = base + q * kStConsumerThreads + tid;
                dst[q] = -1;
                if (it < routed_items) {
                    int pair, i;
                    fdivmod(it, p.fd_qi, pair, i);
                    const int e = s_pair_e[pair];
                    if (e >= p.expert_base && e < p.expert_base + p.local_experts) {
                        val[q] = __ldcg(reinterpret_cast<const float4*>(p.act + (size_t)pair * p.I + 4 * i));
                        dst[q] = pair * p.I + 4 * i;
                    }
                } else if (it < items) {
                    int b, i;
                    fdivmod(it - routed_items, p.fd_qis, b, i);
                    val[q] = __ldcg(reinterpret_cast<const float4*>(p.sact + (size_t)b * p.Is + 4 * i));
                    dst[q] = (int)shared_base + b * p.Is + 4 * i;
                }
            }
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (dst[q] >= 0) *reinterpret_cast<float4*>(actf + dst[q]) = val[q];
        }
    }
    named_barrier(1, kStConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 8);

    // ---- down rows.  part[slot][row]: slot < npairs routed pairs, then one per token (shared expert).
    //      Blocks in order: the shared expert's, then one per distinct expert; their rows form one list
    //      that is cut into twelve equal runs, one per warp, so the phase is one pass over the weights. ----
    {
        const int has_shared = p.Is > 0 ? 1 : 0;
        const int total = (n_unique + has_shared) * hr;
        const int f0 = (total * warp) / kStConsumerWarps, f1 = (total * (warp + 1)) / kStConsumerWarps;
        const int nchI = p.I >> 3, nchIs = p.Is >> 3;
        // block number `ub` (0 = shared when there is one) at `blk`: this warp's rows of it, if any
        auto do_block = [&](int ub, const T* blk, unsigned long long* bar) {
            const int base = ub * hr;
            const int lo = max(f0, base) - base, hi = min(f1, base + hr) - base;
            if (lo >= hi) return;
            if (bar && ok) ok = mbar_wait(bar, 0, &s_abort);
            if (!ok) return;
            const bool shared = has_shared && ub == 0;
            const unsigned long long m = shared ? ((NT > 1 && p.ntok > 1) ? 3ull : 1ull) : s_uniq_m[ub - has_shared];
            const int q0 = __ffsll((long long)m) - 1;
            const unsigned long long m1 = m & (m - 1);
            const int q1 = m1 ? __ffsll((long long)m1) - 1 : q0;
            const bool two = (NT > 1 && m1 != 0ull);
            const float* abase = shared ? actf + shared_base : actf;
            const int len = shared ? p.Is : p.I;
            const int nch = shared ? nchIs : nchI;
            float* pq = shared ? part + npairs * p.hr_max : part;
            const float* a0 = abase + (size_t)q0 * len;
            const float* a1 = abase + (size_t)q1 * len;
#pragma unroll 1
            for (int r = lo; r < hi; r += kStRowBatch) {
                if (two) down_rows<T, NT>(blk, r, min(hi, r + kStRowBatch), nch, a0, a1, pq + q0 * p.hr_max, pq + q1 * p.hr_max, lane);
                else down_rows<T, 1>(blk, r, min(hi, r + kStRowBatch), nch, a0, a0, pq + q0 * p.hr_max, pq, lane);
            }
        };
        if (has_shared) do_block(0, sdown_buf, sdown_bar);
        const int nd = min(p.nded, n_unique);
#pragma unroll 1
        for (int j = 0; j < nd; ++j) do_block(j + has_shared, reinterpret_cast<const T*>(ded + (size_t)j * p.unit_bytes), &ded_bar[j]);
        if (tracer) trace_stamp(p.ctl, 13);
        // the rest arrives through the ring; the first of these chunks is the one the gate/up loop stopped at
#pragma unroll 1
        for (int done = nd; done < n_unique && ok;) {
            if (d.x != kChunkDown) { ok = false; break; }  // cannot happen: the producer sends exactly these chunks
#pragma unroll 1
            for (int q = 0; q < d.z; ++q)
                do_block(d.y + q + has_shared, reinterpret_cast<const T*>(ring + (size_t)stage * kStStageBytes + (size_t)q * p.unit_bytes), nullptr);
            done += d.z;
            release_chunk();
            if (done < n_unique) wait_chunk();
        }
        if (tracer) trace_stamp(p.ctl, 14);
        if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    }
    named_barrier(1, kStConsumerThreads);
    if (tid == 0) cta_stamp(p.ctl, cta, 2);
    if (*(volatile int*)&s_abort != 0) return;

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
                const int pair = b * p.K + k;
                const int e = s_pair_e[pair];
                if (e >= p.expert_base && e < p.expert_base + p.local_experts) v = fmaf(s_pair_w[pair], part[pair * p.hr_max + j], v);
            }
            if (p.Is > 0) v += part[(npairs + b) * p.hr_max + j];
            const size_t o = (size_t)b * p.H + h0 + j;
            if (exchange) {
                comm_put(p.comm, step, o, v);  // this rank's share of element o, to every rank
                // the same thread collects the ranks' shares of its element, in rank order
                if (comm_get_sum(p.comm, p.ctl, step, o, &v)) out[o] = from_float<T>(v + resid);
            } else if (p.partial_out) {
                p.partial_out[o] = v;
            } else {
                out[o] = from_float<T>(v + resid);
            }
        }
    }
    // every CTA read the step counter at entry, long before any CTA can get here
    if (exchange && cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);
    if (tracer) {
        trace_stamp(p.ctl, 9);
        p.ctl->trace[23] = (unsigned long long)clock64();
    }
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------

// Launches the stream kernel when the call suits it (one or two tokens, 2-byte dtype, aligned shapes) and
// sets *handled; otherwise leaves *handled false (no error) so that the caller tries the other kernels.
int moe_decode_stream_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                             bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    if (a->batch < 1 || a->batch > kStMaxTokens) return MK36_OK;
    const int H = a->hidden, E = a->experts, K = a->top_k, I = a->intermediate, Is = a->shared_intermediate;
    const int ntok = a->batch;
    if (K <= 0 || K > 32 || ntok * K > kStMaxPairs || I <= 0 || Is < 0 || E <= 0 || E > 32 * kStTopkPerLane || ntok * E > kTagSlots) return MK36_OK;
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
    if (rows_max * kStMaxTokens > kStMaxPublish) return MK36_OK;
    if (H > 8 * kStConsumerThreads) return MK36_OK;  // one 16-byte piece of x per consumer thread
    const size_t unit_bytes = (size_t)hr_max * I * 2;
    if (unit_bytes > (size_t)kStStageBytes || (size_t)hr_max * Is * 2 > 65536) return MK36_OK;
    if ((long long)ntok * K * (I / pr) * 2 >= (1ll << 31)) return MK36_OK;

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
    const int pairs = ntok * K;
    p.off_bars = take((2 * kStMaxStages + kStMaxDed + 2) * 8, 16);
    p.off_desc = take(kStMaxStages * 16, 16);
    p.off_uniq_e = take(kStMaxPairs * 4, 16);
    p.off_uniq_m = take(kStMaxPairs * 8, 16);
    p.off_pair_e = take(kStMaxPairs * 4, 16);
    p.off_pair_w = take(kStMaxPairs * 4, 16);
    p.off_part = take((size_t)(pairs + ntok) * hr_max * 4, 16);
    p.off_sdown = take((size_t)hr_max * Is * 2, 128);
    const size_t xs_bytes = (size_t)ntok * H * 2;
    const size_t act_bytes = ((size_t)pairs * I + (size_t)ntok * Is) * 4;
    p.off_act = take(xs_bytes > act_bytes ? xs_bytes : act_bytes, 128);
    p.off_ring = take(0, 128);
    const long long room = (long long)dev->max_smem_optin - (long long)off - 1024;  // 1024: the kernel's static shared memory
    // Ring depth against slots for the down blocks: the ring bounds the bytes in flight while the gate/up rows
    // stream, the slots decide how much of the down projection is already requested when that stream ends.
    int nstages = options().moe_stages > 0 ? options().moe_stages : 4;
    if (nstages > kStMaxStages) nstages = kStMaxStages;
    while (nstages > 2 && (long long)nstages * kStStageBytes + (long long)unit_bytes > room) --nstages;
    if ((long long)nstages * kStStageBytes > room || nstages < 2) return MK36_OK;
    int nded = (int)((room - (long long)nstages * kStStageBytes) / (long long)unit_bytes);
    if (nded > kStMaxDed) nded = kStMaxDed;
    if (nded > pairs) nded = pairs;
    p.off_ded = p.off_ring + nstages * kStStageBytes;
    const size_t smem_bytes = (size_t)p.off_ded + (size_t)nded * unit_bytes;

    const size_t scratch = align_up((size_t)ntok * E * 4, 256) + align_up((size_t)pairs * I * 4, 256) + align_up((size_t)ntok * (Is > 0 ? Is : 1) * 4, 256);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + scratch)
        MK36_FAIL(MK36_ERR_WORKSPACE, "moe_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, kControlBytes + scratch);
    // the mailboxes live at a fixed offset that nothing else writes; a smaller workspace takes the ring kernel
    if (ncta > kMailboxMaxCtas || workspace_bytes < kTaggedEnd) return MK36_OK;

    p.x = a->x;
    p.norm_w = a->norm_weight;
    p.router_w = a->router_weight;
    p.egate = a->expert_gate;
    p.eup = a->expert_up;
    p.edown = a->expert_down;
    p.sgate = a->shared_gate;
    p.sup = a->shared_up;
    p.sdown = a->shared_down;
    p.out = a->out;
    p.indices = reinterpret_cast<long long*>(a->indices);
    p.route_w = a->route_weights;
    p.partial_out = a->partial_out;
    p.ctl = static_cast<Control*>(workspace);
    p.mailbox = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(workspace) + kMailboxOffset);
    unsigned char* sc = static_cast<unsigned char*>(workspace) + kControlBytes + align_up((size_t)ntok * E * 4, 256);
    p.act = reinterpret_cast<float*>(sc);
    sc += align_up((size_t)pairs * I * 4, 256);
    p.sact = reinterpret_cast<float*>(sc);
    p.ntok = ntok; p.H = H; p.E = E; p.K = K; p.I = I; p.Is = Is;
    p.expert_base = a->expert_base;
    p.local_experts = a->local_experts;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    p.nstages = nstages;
    p.nded = nded;
    p.pr = pr;
    p.hr_max = hr_max;
    p.unit_bytes = (int)unit_bytes;
    p.upc = (int)(kStStageBytes / unit_bytes);
    p.deal_static = options().moe_static ? 1 : 0;
    // the last rounds go through the counter so that CTAs whose memory is served faster take more: with four of the
    // seven rounds of a one-token step dealt that way the CTAs reach the grid barrier within 1.3 us of one another
    // (2.9 us with two)
    p.dyn_rounds = options().moe_dyn_rounds > 0 ? options().moe_dyn_rounds : 4;
    // mailboxes as close together as the token count allows (the distance between them made no measurable
    // difference to when the logits are seen: 512, 528 and 2048 words were tried on one GPU)
    p.box_stride = (ntok * E + 511) / 512 * 512;
    p.fd_ncta = make_fastdiv(ncta);
    p.fd_cpe = make_fastdiv(I / pr);
    p.fd_K = make_fastdiv(K);
    p.fd_qi = make_fastdiv(I / 4);
    p.fd_qis = make_fastdiv(Is > 0 ? Is / 4 : 1);
    p.fd_npr = make_fastdiv(H / 8);

    const void* kernel = (a->dtype == MK36_BF16)
                             ? (ntok == 1 ? (const void*)moe_decode_stream_kernel<__nv_bfloat16, 1> : (const void*)moe_decode_stream_kernel<__nv_bfloat16, 2>)
                             : (ntok == 1 ? (const void*)moe_decode_stream_kernel<__half, 1> : (const void*)moe_decode_stream_kernel<__half, 2>);
    {
        const int rc_smem = ensure_dynamic_smem(kernel, smem_bytes);
        if (rc_smem != MK36_OK) return rc_smem;
    }
    void* params[] = {&p};
    const int rc = launch_cooperative(kernel, dim3(ncta), dim3(kStThreads), smem_bytes, stream, params, "moe_decode(stream)");
    if (rc != MK36_OK) return rc;
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
