// Pieces shared by the MoE streaming kernels (moe_decode_stream.cu: one token, two on request;
// moe_decode_batch.cu: two to eight tokens): ring geometry, kernel parameters, the row-pair and
// down-row contractions and the relaxed 64-bit loads / stores of the tagged mailbox words.
#pragma once
#include <cfloat>
#include <climits>

#include "mk36_comm.cuh"
#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kStConsumerWarps = 12;  // 12 + 1 producer: 13 warps are allocated as 16, i.e. 128 registers per thread
constexpr int kStConsumerThreads = kStConsumerWarps * 32;
constexpr int kStThreads = kStConsumerThreads + 32;
constexpr int kStGroups = 3;
constexpr int kStGroupWarps = kStConsumerWarps / kStGroups;
constexpr int kStStageBytes = 32768;  // bulk copies under 16 KB cost bandwidth
constexpr int kStMaxStages = 6;
constexpr int kStMaxDed = 16;         // down-projection blocks with a slot of their own
constexpr int kStMaxTokens = 2;
constexpr int kStMaxPairs = 64;
constexpr int kStMaxRows = 16;        // output rows per CTA
constexpr int kStTopkPerLane = 8;     // register top-k: experts <= 256
constexpr int kStRouterPieces = 2;    // 16-byte pieces of router rows per consumer thread
constexpr int kStRouterSlots = kStRouterPieces * kStConsumerWarps;
constexpr int kStMaxPublish = 8;      // (router row, token) logits one CTA publishes

enum : int { kChunkEnd = 0, kChunkShared = 1, kChunkRouted = 2, kChunkDown = 3 };

struct MoeStreamParams {
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
    unsigned long long* mailbox;  // [boxes][box_stride] tagged logits, one copy per receiving CTA (or group of CTAs)
    int box_stride;               // words per mailbox: tokens x experts rounded up to 512 (at most kTagSlots)
    float* act;   // [ntok*K][I]   silu(gate) * up of the routed pairs
    float* sact;  // [ntok][Is]    same for the shared expert
    int ntok, H, E, K, I, Is;
    int expert_base, local_experts, add_residual;
    float eps;
    int nstages;      // ring depth
    int nded;         // down blocks that get a slot of their own
    int pr;           // (gate, up) pairs per stage
    int hr_max;       // max output rows per CTA
    int unit_bytes;   // hr_max * I * sizeof(T): one expert's block of this CTA's down rows
    int upc;          // down blocks per ring stage
    int deal_static;  // 1: chunk k of CTA c is chunk k * ncta + c, no work counter
    int dyn_rounds;   // rounds at the end of the gate/up stream that are dealt through the work counter
    FastDiv fd_ncta, fd_cpe, fd_K, fd_qi, fd_qis, fd_npr;
    int box_share;    // batch kernel: CTAs that read the same mailbox
    int off_emask;    // batch kernel: per expert, the (token, slot) pairs that chose it
    int off_ring, off_ded, off_sdown, off_act, off_part, off_uniq_e, off_uniq_m, off_pair_e, off_pair_w, off_desc, off_bars;
    CommParams comm;
};

template <typename T>
__device__ __forceinline__ void st_unpack(const uint4& v, float (&f)[8]) {
    Chunk8<T> c;
    c.raw = v;
    unpack8(c, f);
}

// (gate, up) row pair against NV token vectors, all in shared memory.  Lane l reads the 16-byte pieces
// l, l + 32, ... (conflict-free); the warp reduces with shuffles.  Returns {g.x0, u.x0, g.x1, u.x1}.
template <typename T, int NV>
__device__ __noinline__ float4 pair_dot(const T* g, const T* u, const T* x0, const T* x1, int nchunks, int lane) {
    float sg[NV], su[NV];
#pragma unroll
    for (int t = 0; t < NV; ++t) { sg[t] = 0.0f; su[t] = 0.0f; }
#pragma unroll 2
    for (int c = lane; c < nchunks; c += 32) {
        float fg[8], fu[8];
        st_unpack<T>(lds128(g + 8 * c), fg);
        st_unpack<T>(lds128(u + 8 * c), fu);
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            float fx[8];
            st_unpack<T>(lds128((t == 0 ? x0 : x1) + 8 * c), fx);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                sg[t] = fmaf(fg[i], fx[i], sg[t]);
                su[t] = fmaf(fu[i], fx[i], su[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        sg[t] = warp_sum(sg[t]);
        su[t] = warp_sum(su[t]);
    }
    return make_float4(sg[0], su[0], sg[NV - 1], su[NV - 1]);
}

// Rows [r_begin, r_end) (at most kStRowBatch of them) of one down block (rows of `nchunks` 16-byte
// pieces, nchunks <= 64, at `blk` in shared memory) against the fp32 activations of one or two pairs
// (a0, a1 in shared memory), which go into registers first: lane l has pieces l and l + 32.  A row costs one pass over its
// weights and nothing else from shared memory (lane l reads 16-byte piece l of the row: conflict-free;
// a 16 x 8 tensor-core tile over rows that are 1 KB apart would take every fragment load eight-way
// bank-conflicted).  All rows of the batch are in flight together: independent load / FMA / shuffle
// chains, because a warp that did them one after the other would spend its time waiting for its own
// latencies.  Row r's sums go to out0[r] / out1[r].
constexpr int kStRowBatch = 6;
template <typename T, int NV>
__device__ __noinline__ void down_rows(const T* blk, int r_begin, int r_end, int nchunks, const float* a0, const float* a1, float* out0,
                                       float* out1, int lane) {
    // the activation vectors (fp32, shared memory) into registers
    float a[NV][2][8];
#pragma unroll
    for (int t = 0; t < NV; ++t) {
        const float* ap = (t == 0) ? a0 : a1;
#pragma unroll
        for (int q = 0; q < 2; ++q) {
            const int c = lane + 32 * q;
            float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
            if (c < nchunks) {
                v0 = *reinterpret_cast<const float4*>(ap + 8 * c);
                v1 = *reinterpret_cast<const float4*>(ap + 8 * c + 4);
            }
            a[t][q][0] = v0.x; a[t][q][1] = v0.y; a[t][q][2] = v0.z; a[t][q][3] = v0.w;
            a[t][q][4] = v1.x; a[t][q][5] = v1.y; a[t][q][6] = v1.z; a[t][q][7] = v1.w;
        }
    }
    const uint4 zero = make_uint4(0, 0, 0, 0);
    uint4 w0[kStRowBatch], w1[kStRowBatch];
#pragma unroll
    for (int j = 0; j < kStRowBatch; ++j) {
        const int r = r_begin + j;
        const T* w = blk + (size_t)r * nchunks * 8;
        w0[j] = (r < r_end && lane < nchunks) ? lds128(w + 8 * lane) : zero;
        w1[j] = (r < r_end && lane + 32 < nchunks) ? lds128(w + 8 * (lane + 32)) : zero;
    }
    float sv[NV][kStRowBatch];
#pragma unroll
    for (int j = 0; j < kStRowBatch; ++j) {
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
            for (int j = 0; j < kStRowBatch; ++j) sv[t][j] += __shfl_xor_sync(kFullMask, sv[t][j], off);
    }
    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < kStRowBatch; ++j) {
            const int r = r_begin + j;
            if (r < r_end) {
                out0[r] = sv[0][j];
                if (NV > 1) out1[r] = sv[NV - 1][j];
            }
        }
    }
}

__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}

// ---- top-k of up to 256 router logits held eight per lane (expert e = lane + 32 j in slot j) ----
// Keys are order-preserving unsigned images of the fp32 logits (larger logit = larger key, 0 = no
// logit).  Every lane first sorts its eight (key, slot) pairs - a 19-exchange network, all lanes at
// once - so that a selection round is one warp-wide maximum over the lanes' heads and a shift on the
// winning lane: the selection is a chain of dependent warp-wide operations, and its length, not the
// arithmetic, is what a launch of one token waits for.  Order: descending logit, lowest expert
// index on equal logits (mega_kernel_qwen36/reference.py:30-33 selects with torch.topk; the
// oracle fixes the order on ties the same way).
__device__ __forceinline__ void topk_exchange(unsigned& ka, int& ia, unsigned& kb, int& ib) {
    const bool sw = (kb > ka) || (kb == ka && ib < ia);
    const unsigned k0 = sw ? kb : ka, k1 = sw ? ka : kb;
    const int i0 = sw ? ib : ia, i1 = sw ? ia : ib;
    ka = k0; kb = k1; ia = i0; ib = i1;
}

__device__ __forceinline__ unsigned topk_key(unsigned logit_bits) {
    return (logit_bits & 0x80000000u) ? ~logit_bits : (logit_bits | 0x80000000u);
}

__device__ __forceinline__ float topk_logit(unsigned key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}

// Calls emit(round, expert, logit) on the lane that holds round r's winner, for r = 0 .. K - 1.
template <typename Emit>
__device__ __forceinline__ void topk_select(unsigned (&k)[kStTopkPerLane], int K, int lane, Emit&& emit) {
    static_assert(kStTopkPerLane == 8, "the exchange network below sorts eight keys");
    int i[8] = {0, 1, 2, 3, 4, 5, 6, 7};
#define MK36_CE(a, b) topk_exchange(k[a], i[a], k[b], i[b])
    MK36_CE(0, 1); MK36_CE(2, 3); MK36_CE(4, 5); MK36_CE(6, 7);
    MK36_CE(0, 2); MK36_CE(1, 3); MK36_CE(4, 6); MK36_CE(5, 7);
    MK36_CE(1, 2); MK36_CE(5, 6);
    MK36_CE(0, 4); MK36_CE(1, 5); MK36_CE(2, 6); MK36_CE(3, 7);
    MK36_CE(2, 4); MK36_CE(3, 5);
    MK36_CE(1, 2); MK36_CE(3, 4); MK36_CE(5, 6);
#undef MK36_CE
#pragma unroll 1
    for (int r = 0; r < K; ++r) {
        const unsigned kmax = __reduce_max_sync(kFullMask, k[0]);
        bool mine = (k[0] == kmax);
        const unsigned tie = __ballot_sync(kFullMask, mine);
        if (tie & (tie - 1u)) {  // several lanes hold the maximum: the lowest expert index wins
            const unsigned cand = mine ? (unsigned)(lane + 32 * i[0]) : 0xffffffffu;
            mine = (cand == __reduce_min_sync(kFullMask, cand));
        }
        if (mine) {
            emit(r, lane + 32 * i[0], topk_logit(kmax));
#pragma unroll
            for (int j = 0; j + 1 < 8; ++j) {
                k[j] = k[j + 1];
                i[j] = i[j + 1];
            }
            k[7] = 0u;
        }
    }
}

}  // namespace mk36
