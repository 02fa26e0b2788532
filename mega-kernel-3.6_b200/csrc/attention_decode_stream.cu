// Full-attention GQA decode, streaming variant for sm_100a (bf16 / f16, head_dim 64/128/256, up to 8
// query heads per KV head, 1/2/4/8 KV heads).  Same arithmetic as attention_decode_mma.cu (reference:
// mega_kernel_qwen36/reference.py:117-145, fp32 scores and accumulation); what changes is how the
// cache gets to the tensor-core tiles.
//
// The cache is [T, Hkv, D]: the rows of ONE KV head are D elements at a stride of Hkv * D, too small
// for bulk copies, but the rows of ALL KV heads of a run of tokens are one contiguous block.  So a CTA
// owns (batch item, token range) for every KV head, one producer lane brings K and V of 32 KB worth
// of tokens per stage into a shared-memory ring with two 1-D bulk copies (cp.async.bulk completing
// on an mbarrier, each copy into the issuing CTA only), and nothing is staged in registers: 3 stages
// x 64 KB are in flight per SM instead of the 16 KB per warp that register double-buffering allows.
//
// Eight consumer warps: unit u = (16-token tile, KV head) of the CTA's stream goes to warp u mod 8, and
// since the number of KV heads divides 8 a warp always serves the same KV head, so its online soft-max
// state and output accumulators never change owner.  Every warp waits for every stage and releases
// it (all warps see every barrier phase exactly once, in order).  The query heads of the warp's KV
// head are the N side of mma.sync.m16n8k16:
//     S[16 tokens, 8 heads] = K_tile[16, D] . Q^T[D, 8]            (M = tokens, K = channels)
//     O^T[D, 8 heads]      += V_tile^T[D, 16] . P^T[16 tokens, 8]  (M = channels, K = tokens)
// with the fragment conventions of attention_decode_mma.cu (contraction index permuted identically on
// both operands, one 128-bit shared-memory load per fragment, P transposed with movmatrix).
//
// A CTA's tokens need not be contiguous (the online soft-max does not care about order): chunk c of a
// batch item goes to CTA c mod splits for the first rounds and, with one batch item, through a work
// counter afterwards, so that a CTA whose memory is served faster takes more and all CTAs reach the
// merge together.  The producer writes what a stage holds (first token, tokens; none = the stream has
// ended) next to it before it arms the stage.
//
// At the end the warps of a KV head are folded in shared memory (over the ring, which is dead by
// then), the CTA writes its (m, l, o) partials, and the shared merge (one bounded grid barrier)
// combines the splits.
#include <cfloat>

#include "mk36_attention.cuh"
#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kAsConsumerWarps = 8;
constexpr int kAsConsumerThreads = kAsConsumerWarps * 32;
constexpr int kAsThreads = kAsConsumerThreads + 32;
constexpr int kAsTile = 16;
constexpr int kAsMaxStages = 4;
constexpr int kAsStageBytes = 32768;  // of K, and as much of V

struct AttnStreamParams {
    AttnParams a;
    int stage_tokens;  // tokens per stage (multiple of 16): stage_tokens * Hkv * D * 2 = kAsStageBytes
    int nstages;
    int deal;          // 1: the chunks of the (single) batch item are dealt through the work counter
    int off_q, off_bars, off_desc, off_ring;  // byte offsets into dynamic shared memory; the fold buffers lie over the ring
};

template <typename T>
__device__ __forceinline__ void as_mma(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void as_mma<__nv_bfloat16>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                                      unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void as_mma<__half>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                               unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ unsigned as_pack2(float lo, float hi);
template <>
__device__ __forceinline__ unsigned as_pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned as_pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <typename T>
__device__ __forceinline__ float2 as_unpack2(unsigned v);
template <>
__device__ __forceinline__ float2 as_unpack2<__nv_bfloat16>(unsigned v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 as_unpack2<__half>(unsigned v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

__device__ __forceinline__ unsigned as_transpose8x8(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

template <typename T, int D>
__global__ void __launch_bounds__(kAsThreads, 1) attention_decode_stream_kernel(const AttnStreamParams sp) {
    constexpr int NSL = D / 32;   // 32-wide channel slices of the score product
    constexpr int NW = D / 16;    // 32-bit words of V per lane and token = M tiles of the output product
    constexpr int NV4 = D / 64;   // 128-bit loads of V per lane and token
    const AttnParams& p = sp.a;
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_abort;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const bool is_producer = (warp == kAsConsumerWarps);

    T* sq = reinterpret_cast<T*>(smem + sp.off_q);  // [Hkv][8][D] query heads, zero padded to 8 per KV head
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + sp.off_bars);
    unsigned long long* empty_bar = full_bar + kAsMaxStages;
    unsigned char* ring = smem + sp.off_ring;

    const int split = blockIdx.x % p.splits;
    const int b = blockIdx.x / p.splits;
    const int ST = sp.stage_tokens, R = sp.nstages;
    const size_t tok_elems = (size_t)p.Hkv * D;  // elements per token (all KV heads)

    int2* desc = reinterpret_cast<int2*>(smem + sp.off_desc);  // per stage: {first token, tokens}
    const int chunks_all = (p.T + ST - 1) / ST;                // chunks of one batch item

    const bool tracer = (blockIdx.x == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);
    if (tid < 2 * kAsMaxStages) mbar_init(&full_bar[tid], tid < kAsMaxStages ? 1 : kAsConsumerWarps);
    if (tid == 0) s_abort = 0;
    if (tid < 32) mbar_init_fence();
    __syncthreads();

    // =====================================================================================
    // Producer: K and V of a run of tokens are one contiguous block each
    // =====================================================================================
    if (is_producer) {
        if (lane != 0) return;
        if (ld_volatile_s32(&p.ctl->status) != 0) {  // nothing may run on a workspace whose status word is set
            *(volatile int*)&s_abort = 1;
            return;
        }
        const T* kbase = static_cast<const T*>(p.k) + (size_t)b * p.T * tok_elems;
        const T* vbase = static_cast<const T*>(p.v) + (size_t)b * p.T * tok_elems;
        bool ok = true;
        int stage = 0, use = 0;
        // the first rounds are dealt statically (chunk k * splits + split), the rest through the counter
        int static_rounds = chunks_all / p.splits;
        if (sp.deal) static_rounds = max(static_rounds - 2, 0);
        const int dyn_base = static_rounds * p.splits;
        int k = 0;
        int t_next = (k < static_rounds || !sp.deal) ? split : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
        for (;;) {
            const int c = t_next;
            const bool last = c >= chunks_all;
            if (!last) {
                ++k;
                t_next = (k < static_rounds || !sp.deal) ? k * p.splits + split : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
            }
            if (use > 0) ok = mbar_wait(&empty_bar[stage], (unsigned)(use - 1) & 1u, &s_abort);
            if (!ok) break;
            if (last) {
                desc[stage] = make_int2(0, 0);  // an empty chunk: the stream of this CTA has ended
                mbar_arrive(&full_bar[stage]);
                break;
            }
            const int tok0 = c * ST;
            const int ntok = min(ST, p.T - tok0);
            const unsigned bytes = (unsigned)((size_t)ntok * tok_elems * sizeof(T));
            unsigned char* dst = ring + (size_t)stage * 2 * kAsStageBytes;
            desc[stage] = make_int2(tok0, ntok);
            mbar_arrive_expect_tx(&full_bar[stage], 2 * bytes);
            bulk_copy_g2s(dst, kbase + (size_t)tok0 * tok_elems, bytes, &full_bar[stage]);
            bulk_copy_g2s(dst + kAsStageBytes, vbase + (size_t)tok0 * tok_elems, bytes, &full_bar[stage]);
            if (++stage == R) { stage = 0; ++use; }
        }
        if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingProducer);
        return;  // consumers wait on every barrier that was armed: no copy is in flight when the CTA leaves
    }

    // =====================================================================================
    // Consumers
    // =====================================================================================
    // the query heads, grouped by KV head and zero padded to 8 rows per group (one 16-byte load per thread and pass)
    {
        const T* q = static_cast<const T*>(p.q) + (size_t)b * p.Hq * D;
        for (int i = tid * 8; i < p.Hkv * 8 * D; i += kAsConsumerThreads * 8) {
            const int row = i / D, d = i - row * D;
            const int kh = row >> 3, h = row & 7;
            *reinterpret_cast<uint4*>(sq + i) =
                (h < p.group) ? *reinterpret_cast<const uint4*>(q + (size_t)(kh * p.group + h) * D + d) : make_uint4(0, 0, 0, 0);
        }
    }
    named_barrier(1, kAsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 1);

    const int kvh = warp % p.Hkv;                 // the KV head this warp serves
    const int units_per_tile = p.Hkv;             // unit = (tile, KV head); unit u -> warp u mod 8
    const T* myq = sq + (size_t)kvh * 8 * D;

    float o[NW][4];
#pragma unroll
    for (int m = 0; m < NW; ++m) { o[m][0] = 0.f; o[m][1] = 0.f; o[m][2] = 0.f; o[m][3] = 0.f; }
    float mrun[2] = {-INFINITY, -INFINITY};  // running max of heads 2t, 2t+1
    float lrun[2] = {0.0f, 0.0f};            // this lane's share of the running sums
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    bool ok = true;
    int stage = 0, use = 0;
    int unit0 = 0;  // number of the first unit of the current chunk
    for (;;) {
        if (ok) ok = mbar_wait(&full_bar[stage], (unsigned)use & 1u, &s_abort);
        if (!ok) break;
        const int ntok = desc[stage].y;
        if (ntok == 0) break;  // the producer's end mark
        const int ntiles = (ntok + kAsTile - 1) / kAsTile;
        const T* ks = reinterpret_cast<const T*>(ring + (size_t)stage * 2 * kAsStageBytes);
        const T* vs = reinterpret_cast<const T*>(ring + (size_t)stage * 2 * kAsStageBytes + kAsStageBytes);
        // this warp's tiles of the chunk: units unit0 + tile * Hkv + kvh with (unit mod 8) == warp
        for (int tile = 0; tile < ntiles; ++tile) {
            const int unit = unit0 + tile * units_per_tile + kvh;
            if ((unit & (kAsConsumerWarps - 1)) != warp) continue;
            const int lt0 = tile * kAsTile;  // first token of the tile inside the chunk
            // ---- scores: rows g and g+8 of the tile, channels 32*sl + 8t .. of this KV head ----
            float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
            {
                const bool v0 = (lt0 + g) < ntok, v1 = (lt0 + g + 8) < ntok;
                const T* r0 = ks + ((size_t)(lt0 + g) * p.Hkv + kvh) * D + 8 * t;
                const T* r1 = ks + ((size_t)(lt0 + g + 8) * p.Hkv + kvh) * D + 8 * t;
#pragma unroll
                for (int sl = 0; sl < NSL; ++sl) {
                    const uint4 ka = v0 ? lds128(r0 + 32 * sl) : zero4;
                    const uint4 kb = v1 ? lds128(r1 + 32 * sl) : zero4;
                    const uint4 qv = lds128(myq + (size_t)g * D + 32 * sl + 8 * t);
                    as_mma<T>(s0, ka.x, kb.x, ka.y, kb.y, qv.x, qv.y);
                    as_mma<T>(s1, ka.z, kb.z, ka.w, kb.w, qv.z, qv.w);
                }
            }
            float s[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) s[i] = (s0[i] + s1[i]) * p.scale;
            if (lt0 + g >= ntok) { s[0] = -INFINITY; s[1] = -INFINITY; }
            if (lt0 + g + 8 >= ntok) { s[2] = -INFINITY; s[3] = -INFINITY; }

            // ---- online soft-max for heads 2t (s[0], s[2]) and 2t+1 (s[1], s[3]) ----
            float mx0 = fmaxf(s[0], s[2]), mx1 = fmaxf(s[1], s[3]);
#pragma unroll
            for (int off = 4; off < 32; off <<= 1) {
                mx0 = fmaxf(mx0, __shfl_xor_sync(kFullMask, mx0, off));
                mx1 = fmaxf(mx1, __shfl_xor_sync(kFullMask, mx1, off));
            }
            const float mn0 = fmaxf(mrun[0], mx0), mn1 = fmaxf(mrun[1], mx1);
            const float c0 = (mrun[0] == -INFINITY) ? 0.0f : __expf(mrun[0] - mn0);
            const float c1 = (mrun[1] == -INFINITY) ? 0.0f : __expf(mrun[1] - mn1);
            const float p0 = __expf(s[0] - mn0), p1 = __expf(s[1] - mn1), p2 = __expf(s[2] - mn0), p3 = __expf(s[3] - mn1);
            // the normaliser is summed from the probabilities as they enter the product (rounded to the storage dtype)
            const unsigned pk01 = as_pack2<T>(p0, p1), pk23 = as_pack2<T>(p2, p3);
            const float2 r01 = as_unpack2<T>(pk01), r23 = as_unpack2<T>(pk23);
            lrun[0] = lrun[0] * c0 + r01.x + r23.x;
            lrun[1] = lrun[1] * c1 + r01.y + r23.y;
            if (__any_sync(kFullMask, (mn0 != mrun[0]) || (mn1 != mrun[1]))) {
#pragma unroll
                for (int m = 0; m < NW; ++m) {
                    o[m][0] *= c0; o[m][1] *= c1; o[m][2] *= c0; o[m][3] *= c1;
                }
            }
            mrun[0] = mn0;
            mrun[1] = mn1;
            const unsigned b0 = as_transpose8x8(pk01);
            const unsigned b1 = as_transpose8x8(pk23);

            // ---- output: this lane's tokens 2t, 2t+1, 2t+8, 2t+9, channels g*D/8 .. of this KV head ----
            uint4 vreg[4][NV4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
                const int lt = lt0 + 2 * t + (r & 1) + ((r & 2) ? 8 : 0);
                const T* row = vs + ((size_t)lt * p.Hkv + kvh) * D + g * (D / 8);
#pragma unroll
                for (int j = 0; j < NV4; ++j) vreg[r][j] = (lt < ntok) ? lds128(row + 8 * j) : zero4;
            }
#pragma unroll
            for (int m = 0; m < NW; ++m) {
                const unsigned w0 = reinterpret_cast<const unsigned*>(&vreg[0][m / 4])[m % 4];
                const unsigned w1 = reinterpret_cast<const unsigned*>(&vreg[1][m / 4])[m % 4];
                const unsigned w2 = reinterpret_cast<const unsigned*>(&vreg[2][m / 4])[m % 4];
                const unsigned w3 = reinterpret_cast<const unsigned*>(&vreg[3][m / 4])[m % 4];
                as_mma<T>(o[m], __byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632), __byte_perm(w2, w3, 0x5410),
                          __byte_perm(w2, w3, 0x7632), b0, b1);
            }
        }
        // every warp releases every stage
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == R) { stage = 0; ++use; }
        unit0 += ((ST / kAsTile) * units_per_tile);  // all chunks but the last are full, and the last one's successor is never used
    }
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    if (tracer) trace_stamp(p.ctl, 3);
    // sums over the eight lanes that share a head pair
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        lrun[0] += __shfl_xor_sync(kFullMask, lrun[0], off);
        lrun[1] += __shfl_xor_sync(kFullMask, lrun[1], off);
    }

    // ---- fold the warps (the ring is dead: every stage has been released by every warp) ----
    named_barrier(1, kAsConsumerThreads);
    // Row layout of the fold buffer: channel ch of a head sits at ch + ch / 32 (one float of padding per 32) and
    // a head's row is kFoldRow floats long, chosen so that the 32 lanes of a store (8 channel groups g x 4 head
    // pairs t) fall into 32 different banks: g moves by D / 8 channels, t by two rows.
    constexpr int kFoldRow = (D == 256) ? 268 : (D == 128 ? 134 : 81);  // >= D + D / 32; 2 * kFoldRow mod 32 = 24, 12, 2
    float* s_o = reinterpret_cast<float*>(ring);                     // [warps][8][kFoldRow]
    float* s_m = s_o + (size_t)kAsConsumerWarps * 8 * kFoldRow;      // [warps][8]
    float* s_l = s_m + kAsConsumerWarps * 8;                         // [warps][8]
    float* s_f = s_l + kAsConsumerWarps * 8;                         // [Hkv][8] folded maxima
    float* wo = s_o + (size_t)warp * 8 * kFoldRow;
#pragma unroll
    for (int m = 0; m < NW; ++m) {
        const int ch = g * (D / 8) + 2 * m;
        const int pos = ch + (ch >> 5), pos1 = (ch + 1) + ((ch + 1) >> 5);
        wo[(2 * t) * kFoldRow + pos] = o[m][0];
        wo[(2 * t + 1) * kFoldRow + pos] = o[m][1];
        wo[(2 * t) * kFoldRow + pos1] = o[m][2];
        wo[(2 * t + 1) * kFoldRow + pos1] = o[m][3];
    }
    if (g == 0) {
        s_m[warp * 8 + 2 * t] = mrun[0];
        s_m[warp * 8 + 2 * t + 1] = mrun[1];
        s_l[warp * 8 + 2 * t] = lrun[0];
        s_l[warp * 8 + 2 * t + 1] = lrun[1];
    }
    named_barrier(1, kAsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 4);
    // per (warp, head) rescale factors; only warps of the same KV head meet (warp mod Hkv)
    float f_sc = 0.0f, f_lw = 0.0f, f_mm = 0.0f;
    if (tid < 8 * kAsConsumerWarps) {
        const int w = tid >> 3, h = tid & 7;
        float mm = -INFINITY;
        for (int w2 = w % p.Hkv; w2 < kAsConsumerWarps; w2 += p.Hkv) mm = fmaxf(mm, s_m[w2 * 8 + h]);
        const float mw = s_m[tid];
        f_sc = (mw == -INFINITY) ? 0.0f : __expf(mw - mm);
        f_lw = s_l[tid] * f_sc;
        f_mm = mm;
    }
    named_barrier(1, kAsConsumerThreads);
    if (tid < 8 * kAsConsumerWarps) {
        s_l[tid] = f_lw;  // scaled share of the sum
        s_m[tid] = f_sc;  // factor for the outputs
        if ((tid >> 3) < p.Hkv) s_f[tid] = f_mm;  // warp w < Hkv serves KV head w: slot [w][h]
    }
    named_barrier(1, kAsConsumerThreads);
    // a warp takes whole (KV head, head) rows, lane l the channels 4 l .. 4 l + 3 (+ 128): no division in the loop
    for (int row = warp; row < p.Hkv * 8; row += kAsConsumerWarps) {
        const int kh = row >> 3, h = row & 7;
        if (h >= p.group) continue;
        const int hq = kh * p.group + h;
        const size_t pi = ((size_t)b * p.Hq + hq) * p.splits + split;
#pragma unroll
        for (int d = 4 * lane; d < D; d += 128) {
            const int pos = d + (d >> 5);  // the four channels lie in one 32-channel block
            float acc[4] = {0.f, 0.f, 0.f, 0.f};
            for (int w = kh; w < kAsConsumerWarps; w += p.Hkv) {  // the warps that served this KV head
                const float sc = s_m[w * 8 + h];
                const float* src = s_o + ((size_t)w * 8 + h) * kFoldRow + pos;
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[i] = fmaf(sc, src[i], acc[i]);
            }
            *reinterpret_cast<float4*>(p.part_o + pi * D + d) = make_float4(acc[0], acc[1], acc[2], acc[3]);
        }
        if (lane == 0) {
            float lsum = 0.0f;
            for (int w = kh; w < kAsConsumerWarps; w += p.Hkv) lsum += s_l[w * 8 + h];
            p.part_m[pi] = s_f[kh * 8 + h];
            p.part_l[pi] = lsum;
        }
    }
    if (tracer) trace_stamp(p.ctl, 5);

    // ---- merge the splits: one bounded grid barrier, then every warp of the grid takes items.  The producer
    //      warp has left, so the barrier helpers that sync the whole CTA cannot be used here. ----
    named_barrier(1, kAsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 8);
    if (tid == 0) {
        bool fine = (*(volatile int*)&s_abort == 0);
        if (fine) {
            const unsigned target = barrier_arrive(p.ctl, gridDim.x, 0);
            fine = barrier_wait(p.ctl, target, kStatusAttnBarrier);
            if (fine) barrier_finish(p.ctl, gridDim.x);
        }
        s_flag = fine ? 1 : 0;
    }
    named_barrier(1, kAsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 7);
    if (!s_flag) return;
    attention_merge_items<T>(p, blockIdx.x * kAsConsumerWarps + warp, gridDim.x * kAsConsumerWarps, lane);
    if (tracer) trace_stamp(p.ctl, 6);
}

namespace {

template <typename T>
const void* stream_kernel_for(int d) {
    switch (d) {
        case 64: return (const void*)attention_decode_stream_kernel<T, 64>;
        case 128: return (const void*)attention_decode_stream_kernel<T, 128>;
        case 256: return (const void*)attention_decode_stream_kernel<T, 256>;
        default: return nullptr;
    }
}

}  // namespace

// Launches the streaming variant when the shapes suit it and sets *handled; otherwise leaves *handled false
// (no error) and the caller tries the other kernels.
int attention_decode_stream_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    const int D = a->head_dim, Hkv = a->kv_heads, group = a->query_heads / a->kv_heads;
    if (group > 8 || (D != 64 && D != 128 && D != 256)) return MK36_OK;
    if (Hkv != 1 && Hkv != 2 && Hkv != 4 && Hkv != 8) return MK36_OK;  // a warp keeps its KV head: Hkv divides the warp count
    const size_t tok_bytes = (size_t)Hkv * D * 2;
    if (tok_bytes * kAsTile > (size_t)kAsStageBytes) return MK36_OK;
    const int stage_tokens = (int)(kAsStageBytes / tok_bytes) / kAsTile * kAsTile;
    const void* ptrs[] = {a->q, a->k_cache, a->v_cache};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const void* kernel = (a->dtype == MK36_BF16) ? stream_kernel_for<__nv_bfloat16>(D) : stream_kernel_for<__half>(D);
    if (!kernel) return MK36_OK;
    const long long max_ctas = dev->sm_count;  // one CTA per SM
    if (a->batch > max_ctas) return MK36_OK;

    AttnStreamParams sp;
    size_t off = 0;
    sp.off_bars = (int)off;
    off += 2 * kAsMaxStages * 8;
    sp.off_desc = (int)off;
    off += kAsMaxStages * 8;
    off = align_up(off, 128);
    sp.off_q = (int)off;
    off += (size_t)Hkv * 8 * D * 2;
    off = align_up(off, 128);
    sp.off_ring = (int)off;
    const size_t fold_bytes = ((size_t)kAsConsumerWarps * 8 * (D + D / 32 + 16) + 2 * kAsConsumerWarps * 8 + 8 * 8) * 4;
    const long long room = (long long)dev->max_smem_optin - (long long)off - 256;
    int nstages = (int)(room / (2 * kAsStageBytes));
    if (nstages > kAsMaxStages) nstages = kAsMaxStages;
    if (nstages < 2 || (size_t)nstages * 2 * kAsStageBytes < fold_bytes) return MK36_OK;
    sp.nstages = nstages;
    sp.stage_tokens = stage_tokens;
    const size_t smem = off + (size_t)nstages * 2 * kAsStageBytes;
    {
        const int rc_smem = ensure_dynamic_smem(kernel, smem);
        if (rc_smem != MK36_OK) return rc_smem;
    }
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "full_attention_decode: workspace is NULL or not 256-byte aligned");

    int batch_per_launch = (int)max_ctas;
    if (batch_per_launch > a->batch) batch_per_launch = a->batch;
    auto splits_for = [&](int nb) {
        long long splits = max_ctas / nb;
        const long long by_len = (a->seq_len + kAsTile - 1) / kAsTile;  // at least one tile per CTA
        if (splits > by_len) splits = by_len;
        if (splits > kAttnMergeMaxSplits) splits = kAttnMergeMaxSplits;
        return splits < 1 ? 1ll : splits;
    };
    auto scratch_for = [&](int nb, long long splits) {
        const size_t heads = (size_t)nb * a->query_heads;
        return align_up(heads * splits * D * 4, 256) + 2 * align_up(heads * splits * 4, 256);
    };
    // One CTA per SM for all KV heads means more splits, hence more partial rows, than the other kernels need.
    // Every launch of the call must fit before the first one is made; a workspace that is too small for this
    // kernel is not an error, the tensor-core kernel with its smaller plan takes the call.
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        const int nb = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        if (workspace_bytes < kControlBytes + scratch_for(nb, splits_for(nb))) return MK36_OK;
    }
    const size_t es = 2;
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        const int nb = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        const long long splits = splits_for(nb);
        const size_t heads = (size_t)nb * a->query_heads;
        AttnParams& p = sp.a;
        p.q = static_cast<const unsigned char*>(a->q) + (size_t)b0 * a->query_heads * D * es;
        p.k = static_cast<const unsigned char*>(a->k_cache) + (size_t)b0 * a->seq_len * Hkv * D * es;
        p.v = static_cast<const unsigned char*>(a->v_cache) + (size_t)b0 * a->seq_len * Hkv * D * es;
        p.out = static_cast<unsigned char*>(a->out) + (size_t)b0 * a->query_heads * D * es;
        p.ctl = static_cast<Control*>(workspace);
        unsigned char* sc = static_cast<unsigned char*>(workspace) + kControlBytes;
        p.part_o = reinterpret_cast<float*>(sc);
        sc += align_up(heads * splits * D * 4, 256);
        p.part_m = reinterpret_cast<float*>(sc);
        sc += align_up(heads * splits * 4, 256);
        p.part_l = reinterpret_cast<float*>(sc);
        p.B = nb;
        p.Hq = a->query_heads;
        p.Hkv = Hkv;
        p.D = D;
        p.T = a->seq_len;
        p.group = group;
        p.subgroups = 1;
        p.splits = (int)splits;
        p.scale = a->scale;
        // one work counter: one batch item; and only where the counter has something to balance (with few chunks per
        // CTA the round trips to the counter would cost more than the imbalance)
        sp.deal = (nb == 1 && !options().moe_static && (a->seq_len + stage_tokens - 1) / stage_tokens >= 3 * splits) ? 1 : 0;
        const unsigned grid = (unsigned)((long long)nb * splits);
        void* params[] = {&sp};
        const int rc = launch_cooperative(kernel, dim3(grid), dim3(kAsThreads), smem, stream, params, "full_attention_decode(stream)");
        if (rc != MK36_OK) return rc;
    }
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
