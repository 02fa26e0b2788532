// Decode-time projection: out[b, :] = W . (RMSNorm(x[b, :]) or x[b, :]) (+ residual[b, :]) for one to
// eight tokens, bf16 / f16, with an optional arg-max over the output row (the language-model head).
//
// These are the `linear`, `linear_residual` and `lm_head` tasks of the decode task graph
// (mega_kernel_qwen36/mpk_graph.py:352-398, 418-427, 496-514): the reference's planner names them but
// the reference has no kernel for them (its decode layer takes q, k and v as inputs,
// mega_kernel_qwen36/ops.py:701-748).  The arithmetic follows the formulas the reference uses
// everywhere else: `rms_norm` (mega_kernel_qwen36/reference.py:10-13, result rounded to the input
// dtype), fp32 accumulation, one rounding of the result after the residual was added.
//
// A weight-streaming kernel like the dense FFN's, but without any cross-CTA dependency: a CTA owns
// every `gridDim.x`-th chunk of consecutive weight rows, the producer warp starts the bulk copies of
// its chunks at kernel entry (the weights do not depend on x), and the consumers normalise x into
// shared memory while the first chunks are in flight.  No grid barrier, so an ordinary launch.
//
//   chunk = as many whole rows as fit 32 KB (8 rows at an inner dimension of 2048); row r of chunk k
//   is contracted by warp (k * rows + r) % 8 against one or two tokens; with more tokens a warp takes four
//   rows and four tokens at a time (rows4_dot4);
//   every consumer warp observes and releases every chunk (see moe_decode_stream.cu).
//
// Arg-max: every warp keeps the best (value, row) of the rows it produced per token, on the rounded
// output value with the lower row index winning ties (what arg-max over the stored output would
// give); CTA-wide and then grid-wide maxima go through 64-bit atomic maxima of {ordered value,
// ~row}; the last CTA to leave turns the winners into indices and clears the slots.
#include "mk36_mma.cuh"
#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kLinConsumerWarps = 8;
constexpr int kLinConsumerThreads = kLinConsumerWarps * 32;
constexpr int kLinThreads = kLinConsumerThreads + 32;
constexpr int kLinStageBytes = 32768;
constexpr int kLinMaxStages = 6;
constexpr int kLinMaxTokens = 8;
constexpr int kLinMmaRows = 16;   // weight rows of one tensor-core tile
constexpr int kLinMaxPieces = 8;  // 16-byte pieces of one token per consumer thread: inner dimension <= 16384

struct LinearParams {
    const void* x;
    const void* norm_w;    // null: x is used as it is
    const void* w;         // [N, K]
    const void* residual;  // null or [ntok, N]
    void* out;             // [ntok, N]
    long long* argmax;     // null or [ntok]
    Control* ctl;
    int ntok, K, N;
    float eps;
    int rows;     // weight rows per chunk
    int nchunks;
    int nstages;
    int mma;      // 1: three to eight tokens on tensor-core instructions (tokens are the eight columns of the tile)
    int off_red;  // tensor-core path: the warps' partial tiles, two buffers
    int lg_ppt;   // log2 of the 16-byte pieces of one token per consumer thread, rounded up to a power of two
    int off_x, off_ring, off_bars;
};

template <typename T>
__device__ __forceinline__ void lin_unpack(const uint4& v, float (&f)[8]) {
    Chunk8<T> c;
    c.raw = v;
    unpack8(c, f);
}

// One weight row against NV token vectors, all in shared memory; lane l reads the 16-byte pieces
// l, l + 32, ... of each (conflict-free).
template <typename T, int NV>
__device__ __forceinline__ void row_dot(const T* w, const T* x, size_t xstride, int nch, int lane, float (&s)[NV]) {
    // eight independent accumulators per token: the dependent chain is one FMA per piece, not eight
    float acc[NV][8];
#pragma unroll
    for (int t = 0; t < NV; ++t)
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[t][i] = 0.0f;
#pragma unroll 2
    for (int c = lane; c < nch; c += 32) {
        float fw[8];
        lin_unpack<T>(lds128(w + 8 * c), fw);
#pragma unroll
        for (int t = 0; t < NV; ++t) {
            float fx[8];
            lin_unpack<T>(lds128(x + (size_t)t * xstride + 8 * c), fx);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[t][i] = fmaf(fw[i], fx[i], acc[t][i]);
        }
    }
#pragma unroll
    for (int t = 0; t < NV; ++t)
        s[t] = ((acc[t][0] + acc[t][1]) + (acc[t][2] + acc[t][3])) + ((acc[t][4] + acc[t][5]) + (acc[t][6] + acc[t][7]));
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int t = 0; t < NV; ++t) s[t] += __shfl_xor_sync(kFullMask, s[t], off);
    }
}

// Up to four consecutive weight rows against four token vectors: every 16-byte piece of a token is read once
// for the four rows and every piece of a row once for the four tokens, which keeps the shared-memory traffic
// at twice the weight bytes (one row against four tokens read five pieces per weight piece and was bound by
// shared-memory bandwidth).  Rows beyond `nrows` repeat the last row; their sums are not used.
template <typename T>
__device__ __forceinline__ void rows4_dot4(const T* w, size_t wstride, int nrows, const T* x, size_t xstride, int nch, int lane,
                                           float (&s)[4][4]) {
#pragma unroll
    for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int t = 0; t < 4; ++t) s[r][t] = 0.0f;
    const T* wr[4];
#pragma unroll
    for (int r = 0; r < 4; ++r) wr[r] = w + (size_t)min(r, nrows - 1) * wstride;
#pragma unroll 1
    for (int c = lane; c < nch; c += 32) {
        float fx[4][8];
#pragma unroll
        for (int t = 0; t < 4; ++t) lin_unpack<T>(lds128(x + (size_t)t * xstride + 8 * c), fx[t]);
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            float fw[8];
            lin_unpack<T>(lds128(wr[r] + 8 * c), fw);
#pragma unroll
            for (int t = 0; t < 4; ++t)
#pragma unroll
                for (int i = 0; i < 8; ++i) s[r][t] = fmaf(fw[i], fx[t][i], s[r][t]);
        }
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int t = 0; t < 4; ++t) s[r][t] += __shfl_xor_sync(kFullMask, s[r][t], off);
    }
}

__device__ __forceinline__ unsigned long long argmax_key(float v, int row) {
    const unsigned bits = __float_as_uint(v);
    const unsigned key = (bits & 0x80000000u) ? ~bits : (bits | 0x80000000u);
    return ((unsigned long long)key << 32) | (unsigned long long)(0xffffffffu - (unsigned)row);
}

template <typename T>
__global__ void __launch_bounds__(kLinThreads, 1) linear_decode_kernel(const LinearParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_abort;
    __shared__ int s_dirty;  // the workspace's status word was set at entry: nothing is computed or stored
    __shared__ float s_red[2][kLinConsumerWarps][kLinMaxPieces];
    __shared__ unsigned long long s_best[kLinMaxTokens];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kLinConsumerWarps);

    T* xs = reinterpret_cast<T*>(smem + p.off_x);
    unsigned char* ring = smem + p.off_ring;
    unsigned long long* full_bar = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_bar = full_bar + kLinMaxStages;
    const int R = p.nstages;
    const size_t rowK = (size_t)p.K;
    const int my_chunks = (p.nchunks - cta + ncta - 1) / ncta;  // chunks cta, cta + ncta, ...

    if (tid == 0 && cta == 0) trace_stamp(p.ctl, 0);
    if (tid < 2 * kLinMaxStages) mbar_init(&full_bar[tid], tid >= kLinMaxStages ? kLinConsumerWarps : 1);
    if (tid < kLinMaxTokens) s_best[tid] = 0ull;
    if (tid == 0) {
        s_abort = 0;
        s_dirty = 0;
    }
    if (tid < 32) mbar_init_fence();
    __syncthreads();

    // =====================================================================================
    // Producer warp: this CTA's chunks, in order, as stages come free
    // =====================================================================================
    if (is_producer) {
        if (lane != 0) return;
        bool ok = true;
        int stage = 0, use = 0;
#pragma unroll 1
        for (int k = 0; k < my_chunks && ok; ++k) {
            const int c = cta + k * ncta;
            const int first = c * p.rows;
            const int count = min(p.rows, p.N - first);
            if (use > 0) ok = mbar_wait(&empty_bar[stage], (unsigned)(use - 1) & 1u, &s_abort);
            if (!ok) break;
            const unsigned bytes = (unsigned)((size_t)count * rowK * sizeof(T));
            mbar_arrive_expect_tx(&full_bar[stage], bytes);
            bulk_copy_g2s(ring + (size_t)stage * kLinStageBytes, static_cast<const T*>(p.w) + (size_t)first * rowK, bytes, &full_bar[stage]);
            if (++stage == R) { stage = 0; ++use; }
        }
        if (!ok) atomicCAS(&p.ctl->status, 0, kStatusLinearProducer);
        // consumers wait on every barrier that was armed, so no copy is in flight when the CTA leaves
        return;
    }

    // =====================================================================================
    // Consumer warps
    // =====================================================================================
    // the status word: requested now, looked at after x is in shared memory.  On a workspace whose status is set
    // nothing is computed or stored; the copies the producer has started are still waited for.
    int dirty = 0;
    if (tid == 0) dirty = ld_volatile_s32(&p.ctl->status);

    // ---- x into shared memory as T, normalised when a norm weight is given.  A thread owns eight register
    //      slots: slot j holds piece (tid + (j % ppt) * 256) of token (first + j / ppt), ppt = pieces of one
    //      token per thread rounded up to a power of two, so that as many tokens as fit are loaded, reduced and
    //      normalised in one pass with one block-wide exchange (the loads of x and of the norm weight are all
    //      issued before anything waits). ----
    if (p.ntok == 1) {
        // one token: pieces tid, tid + 256, ... of x and of the norm weight, one block-wide sum
        const int npieces = p.K >> 3;
        const T* x = static_cast<const T*>(p.x);
        uint4 xv[kLinMaxPieces], wv[kLinMaxPieces];
#pragma unroll
        for (int i = 0; i < kLinMaxPieces; ++i) {
            const int piece = tid + i * kLinConsumerThreads;
            xv[i] = make_uint4(0, 0, 0, 0);
            wv[i] = make_uint4(0, 0, 0, 0);
            if (i < (1 << p.lg_ppt) && piece < npieces) {
                xv[i] = *reinterpret_cast<const uint4*>(x + 8 * piece);
                if (p.norm_w) wv[i] = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + 8 * piece);
            }
        }
        float rstd = 1.0f;
        if (p.norm_w) {
            float ss = 0.0f;
#pragma unroll
            for (int i = 0; i < kLinMaxPieces; ++i) {
                if (i < (1 << p.lg_ppt)) {
                    float f[8];
                    lin_unpack<T>(xv[i], f);
#pragma unroll
                    for (int q = 0; q < 8; ++q) ss = fmaf(f[q], f[q], ss);
                }
            }
            ss = warp_sum(ss);
            if (lane == 0) s_red[0][warp][0] = ss;
            named_barrier(1, kLinConsumerThreads);
            float tot = 0.0f;
#pragma unroll
            for (int w = 0; w < kLinConsumerWarps; ++w) tot += s_red[0][w][0];
            rstd = 1.0f / sqrtf(tot / (float)p.K + p.eps);
        }
#pragma unroll
        for (int i = 0; i < kLinMaxPieces; ++i) {
            const int piece = tid + i * kLinConsumerThreads;
            if (i < (1 << p.lg_ppt) && piece < npieces) {
                if (p.norm_w) {
                    float f[8], g[8];
                    lin_unpack<T>(xv[i], f);
                    lin_unpack<T>(wv[i], g);
                    T o[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) o[q] = from_float<T>(__fmul_rn(__fmul_rn(f[q], rstd), g[q]));
                    *reinterpret_cast<uint4*>(xs + 8 * piece) = *reinterpret_cast<const uint4*>(o);
                } else {
                    *reinterpret_cast<uint4*>(xs + 8 * piece) = xv[i];
                }
            }
        }
        if (p.mma) {
            for (int i = tid; i < (kLinMaxTokens - 1) * npieces; i += kLinConsumerThreads)
                *reinterpret_cast<uint4*>(xs + rowK + 8 * (size_t)i) = make_uint4(0, 0, 0, 0);
        }
        if (tid == 0 && dirty != 0) s_dirty = 1;
        named_barrier(1, kLinConsumerThreads);
    } else {
        const int npieces = p.K >> 3;
        const T* x = static_cast<const T*>(p.x);
        const int lg = p.lg_ppt, ppt = 1 << lg;
        const int per_pass = kLinMaxPieces >> lg;  // tokens per pass
        int parity = 0;
#pragma unroll 1
        for (int first_tok = 0; first_tok < p.ntok; first_tok += per_pass, parity ^= 1) {
            uint4 xv[kLinMaxPieces], wv[kLinMaxPieces];
#pragma unroll
            for (int j = 0; j < kLinMaxPieces; ++j) {
                const int b = first_tok + (j >> lg);
                const int piece = tid + (j & (ppt - 1)) * kLinConsumerThreads;
                const bool live = b < p.ntok && piece < npieces;
                xv[j] = make_uint4(0, 0, 0, 0);
                wv[j] = make_uint4(0, 0, 0, 0);
                if (live) {
                    xv[j] = *reinterpret_cast<const uint4*>(x + (size_t)b * rowK + 8 * piece);
                    if (p.norm_w) wv[j] = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + 8 * piece);
                }
            }
            if (p.norm_w == nullptr) {
#pragma unroll
                for (int j = 0; j < kLinMaxPieces; ++j) {
                    const int b = first_tok + (j >> lg);
                    const int piece = tid + (j & (ppt - 1)) * kLinConsumerThreads;
                    if (b < p.ntok && piece < npieces) *reinterpret_cast<uint4*>(xs + (size_t)b * rowK + 8 * piece) = xv[j];
                }
                continue;
            }
            float ssj[kLinMaxPieces];
#pragma unroll
            for (int j = 0; j < kLinMaxPieces; ++j) {
                float f[8];
                lin_unpack<T>(xv[j], f);
                float a = 0.0f;
#pragma unroll
                for (int q = 0; q < 8; ++q) a = fmaf(f[q], f[q], a);
                ssj[j] = a;
            }
            float sst[kLinMaxPieces];  // per token of the pass
#pragma unroll
            for (int tk = 0; tk < kLinMaxPieces; ++tk) {
                float a = 0.0f;
#pragma unroll
                for (int j = 0; j < kLinMaxPieces; ++j) a += ((j >> lg) == tk) ? ssj[j] : 0.0f;
                sst[tk] = a;
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                for (int tk = 0; tk < kLinMaxPieces; ++tk) sst[tk] += __shfl_xor_sync(kFullMask, sst[tk], off);
            }
            if (lane < kLinMaxPieces) {
                float v = sst[0];
#pragma unroll
                for (int tk = 1; tk < kLinMaxPieces; ++tk)
                    if (lane == tk) v = sst[tk];
                s_red[parity][warp][lane] = v;
            }
            named_barrier(1, kLinConsumerThreads);
            float rstd[kLinMaxPieces];
#pragma unroll
            for (int tk = 0; tk < kLinMaxPieces; ++tk) {
                float tot = 0.0f;
#pragma unroll
                for (int w = 0; w < kLinConsumerWarps; ++w) tot += s_red[parity][w][tk];
                rstd[tk] = 1.0f / sqrtf(tot / (float)p.K + p.eps);
            }
#pragma unroll
            for (int j = 0; j < kLinMaxPieces; ++j) {
                const int b = first_tok + (j >> lg);
                const int piece = tid + (j & (ppt - 1)) * kLinConsumerThreads;
                if (b < p.ntok && piece < npieces) {
                    float rs = rstd[0];
#pragma unroll
                    for (int tk = 1; tk < kLinMaxPieces; ++tk)
                        if ((j >> lg) == tk) rs = rstd[tk];
                    float f[8], g[8];
                    lin_unpack<T>(xv[j], f);
                    lin_unpack<T>(wv[j], g);
                    T o[8];
#pragma unroll
                    for (int q = 0; q < 8; ++q) o[q] = from_float<T>(__fmul_rn(__fmul_rn(f[q], rs), g[q]));
                    *reinterpret_cast<uint4*>(xs + (size_t)b * rowK + 8 * piece) = *reinterpret_cast<const uint4*>(o);
                }
            }
            // the next pass writes the other half of s_red; the one after it comes after this pass's barrier
        }
        if (p.mma) {
            // the tile has eight token columns: the ones beyond the batch are zero
            const int npieces8 = (kLinMaxTokens - p.ntok) * (p.K >> 3);
            for (int i = tid; i < npieces8; i += kLinConsumerThreads)
                *reinterpret_cast<uint4*>(xs + (size_t)p.ntok * rowK + 8 * (size_t)i) = make_uint4(0, 0, 0, 0);
        }
        if (tid == 0 && dirty != 0) s_dirty = 1;
        named_barrier(1, kLinConsumerThreads);
    }
    const bool dead = (s_dirty != 0);
    if (tid == 0 && cta == 0) trace_stamp(p.ctl, 1);

    // ---- the chunks ----
    bool ok = true;
    const int nch = p.K >> 3;
    const T* resid = static_cast<const T*>(p.residual);
    T* out = static_cast<T*>(p.out);
    unsigned long long best0 = 0ull, best1 = 0ull;  // lane l < 16: the best of tokens l % 4 and 4 + l % 4 among the rows this lane stored
    int stage = 0, use = 0, slot = 0;  // slot: (rows of the earlier chunks) % warps, the warp of the chunk's first row
#pragma unroll 1
    for (int k = 0; k < my_chunks; ++k) {
        ok = mbar_wait(&full_bar[stage], (unsigned)use & 1u, &s_abort);
        if (!ok) break;
        if (tid == 0 && cta == 0 && k == 1) trace_stamp(p.ctl, 2);
        if (dead) {  // only drain the copies
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == R) { stage = 0; ++use; }
            continue;
        }
        const int first = (cta + k * ncta) * p.rows;
        const int count = min(p.rows, p.N - first);
        const T* sbase = reinterpret_cast<const T*>(ring + (size_t)stage * kLinStageBytes);
        if (p.mma) {
            // Tensor-core path: the chunk's rows (at most sixteen) are the rows of one m16n8k16 tile, the tokens its
            // eight columns.  Warp w contracts the w-th eighth of the inner dimension for the whole tile: per 32-wide
            // slice one 128-bit load per operand (rows g and g + 8 of the weights, token g of x; same permutation of
            // the contraction index on both, see mk36_mma.cuh) and two MMAs.  The eight partial tiles meet in shared
            // memory (two buffers, so one block-wide barrier per chunk), 128 threads finish one output each.
            const int g = lane >> 2, t = lane & 3;
            const int nsl = p.K >> 8;  // 32-wide slices per warp
            float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
            const T* alo = sbase + (size_t)g * rowK + 8 * t;
            const T* ahi = sbase + (size_t)(g + 8) * rowK + 8 * t;
            const T* bx = xs + (size_t)g * rowK + 8 * t;
            const bool lo_live = g < count, hi_live = g + 8 < count;
            const uint4 zero = make_uint4(0, 0, 0, 0);
#pragma unroll 4
            for (int sl = 0; sl < nsl; ++sl) {
                const int kb = (warp * nsl + sl) * 32;
                const uint4 a0 = lo_live ? lds128(alo + kb) : zero;
                const uint4 a1 = hi_live ? lds128(ahi + kb) : zero;
                const uint4 bb = lds128(bx + kb);
                mma_slice32<T>(d0, d1, a0, a1, bb);
            }
            float* red = reinterpret_cast<float*>(smem + p.off_red) + (size_t)(k & 1) * (kLinConsumerWarps * kLinMmaRows * 8);
            float* mine = red + (size_t)warp * (kLinMmaRows * 8);
            *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(d0[0] + d1[0], d0[1] + d1[1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(d0[2] + d1[2], d0[3] + d1[3]);
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);  // the weights of this stage have been read
            if (++stage == R) { stage = 0; ++use; }
            named_barrier(1, kLinConsumerThreads);
            if (tid < kLinMmaRows * 8) {
                const int row = tid >> 3, tok = tid & 7;
                if (row < count && tok < p.ntok) {
                    float v = 0.0f;
#pragma unroll
                    for (int w = 0; w < kLinConsumerWarps; ++w) v += red[(size_t)w * (kLinMmaRows * 8) + tid];
                    const int n = first + row;
                    const size_t o = (size_t)tok * p.N + n;
                    if (resid) v += to_float<T>(resid[o]);
                    const T rounded = from_float<T>(v);
                    out[o] = rounded;
                    if (p.argmax) {
                        const unsigned long long key = argmax_key(to_float<T>(rounded), n);
                        best0 = key > best0 ? key : best0;  // this thread's token is tid % 8 in every chunk
                    }
                }
            }
            continue;
        }
        if (p.ntok > 2) {
            // groups of four rows, four tokens per pass: group g of the chunk goes to warp (slot + g) % warps
            const int groups = (count + 3) >> 2;
            int g = warp - slot;
            if (g < 0) g += kLinConsumerWarps;
#pragma unroll 1
            for (; g < groups; g += kLinConsumerWarps) {
                const int nrows = min(4, count - 4 * g);
                const T* wrow = sbase + (size_t)(4 * g) * rowK;
#pragma unroll 1
                for (int b0 = 0; b0 < p.ntok; b0 += 4) {
                    const int nb = min(4, p.ntok - b0);
                    float s[4][4];
                    rows4_dot4<T>(wrow, rowK, nrows, xs + (size_t)b0 * rowK, rowK, nch, lane, s);
                    const int rr = lane >> 2, tt = lane & 3;
                    if (lane < 16 && rr < nrows && tt < nb) {
                        float v = 0.0f;
#pragma unroll
                        for (int r = 0; r < 4; ++r)
#pragma unroll
                            for (int t = 0; t < 4; ++t)
                                if (rr == r && tt == t) v = s[r][t];
                        const int n = first + 4 * g + rr;
                        const size_t o = (size_t)(b0 + tt) * p.N + n;
                        if (resid) v += to_float<T>(resid[o]);
                        const T rounded = from_float<T>(v);
                        out[o] = rounded;
                        if (p.argmax) {
                            const unsigned long long key = argmax_key(to_float<T>(rounded), n);
                            if (b0 == 0) best0 = key > best0 ? key : best0;
                            else best1 = key > best1 ? key : best1;
                        }
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_bar[stage]);
            if (++stage == R) { stage = 0; ++use; }
            slot += groups;
            while (slot >= kLinConsumerWarps) slot -= kLinConsumerWarps;
            continue;
        }
        int r = warp - slot;
        if (r < 0) r += kLinConsumerWarps;
#pragma unroll 1
        for (; r < count; r += kLinConsumerWarps) {
            const T* wrow = sbase + (size_t)r * rowK;
            const int n = first + r;
            float s[2] = {0.f, 0.f};
            if (p.ntok == 1) {
                float s1[1];
                row_dot<T, 1>(wrow, xs, rowK, nch, lane, s1);
                s[0] = s1[0];
            } else {
                row_dot<T, 2>(wrow, xs, rowK, nch, lane, s);
            }
            if (lane < p.ntok) {
                float v = (lane == 0) ? s[0] : s[1];
                const size_t o = (size_t)lane * p.N + n;
                if (resid) v += to_float<T>(resid[o]);
                const T rounded = from_float<T>(v);
                out[o] = rounded;
                if (p.argmax) {
                    const unsigned long long key = argmax_key(to_float<T>(rounded), n);
                    best0 = key > best0 ? key : best0;
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty_bar[stage]);
        if (++stage == R) { stage = 0; ++use; }
        slot += count;
        while (slot >= kLinConsumerWarps) slot -= kLinConsumerWarps;
    }
    if (!ok) {
        atomicCAS(&p.ctl->status, 0, kStatusLinearConsumer);
        return;
    }
    if (dead) return;
    if (tid == 0 && cta == ncta - 1) trace_stamp(p.ctl, 3);

    // ---- arg-max: CTA-wide maxima first ----
    if (p.argmax && p.mma) {
        if (tid < kLinMmaRows * 8 && best0 != 0ull) atomicMax(&s_best[tid & 7], best0);
    } else if (p.argmax && lane < 16) {
        if (best0 != 0ull) atomicMax(&s_best[lane & 3], best0);
        if (best1 != 0ull) atomicMax(&s_best[4 + (lane & 3)], best1);
    }
    if (!p.argmax) return;  // nothing crosses CTAs: the output rows are stored, the CTA is done
    named_barrier(1, kLinConsumerThreads);
    if (tid < p.ntok && s_best[tid] != 0ull) atomicMax(&p.ctl->best[tid], s_best[tid]);
    if (tid == 0) {
        __threadfence();
        if (atomicAdd(&p.ctl->ticket, 1u) == (unsigned)ncta - 1u) {
            // the last CTA to leave: every CTA's maxima are in; publish and clear for the next kernel
            __threadfence();
            for (int b = 0; b < p.ntok; ++b) {
                const unsigned long long v = atomicExch(&p.ctl->best[b], 0ull);
                p.argmax[b] = (long long)(0xffffffffu - (unsigned)(v & 0xffffffffull));
            }
            p.ctl->ticket = 0u;
            __threadfence();
            trace_stamp(p.ctl, 9);
        }
    }
}

}  // namespace mk36

using namespace mk36;

extern "C" {

size_t mk36_linear_workspace_bytes(const mk36_linear_args* a) {
    (void)a;
    return kControlBytes;
}

int mk36_linear_decode(const mk36_linear_args* a, void* workspace, size_t workspace_bytes, void* stream_) {
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_decode: args is NULL");
    if (!a->x || !a->weight || !a->out) MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_decode: NULL tensor pointer");
    if (a->batch <= 0 || a->in_features <= 0 || a->out_features <= 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_decode: sizes must be positive");
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: dtype must be bf16 or f16");
    const int K = a->in_features, N = a->out_features;
    if (a->batch > kLinMaxTokens) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: at most %d tokens per call (got %d)", kLinMaxTokens, a->batch);
    if (K % 8 != 0 || (size_t)K * 2 > (size_t)kLinStageBytes || K > 8 * kLinMaxPieces * kLinConsumerThreads)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: in_features must be a multiple of 8 and at most %d (got %d)", kLinStageBytes / 2, K);
    const bool p_mma_hint = options().linear_mma > 0 && a->batch >= options().linear_mma && K % 256 == 0;
    if ((size_t)((a->batch > 2 || p_mma_hint) ? kLinMaxTokens : a->batch) * K * 2 > 98304)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: the tokens (eight columns when there are more than two) x in_features x 2 bytes must fit 96 KB of shared memory");
    if ((long long)N * K >= (1ll << 40) || N >= (1 << 30)) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: out_features too large");
    const void* ptrs[] = {a->x, a->weight, a->norm_weight, a->residual, a->out};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_decode: tensors must be 16-byte aligned");
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "linear_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes)
        MK36_FAIL(MK36_ERR_WORKSPACE, "linear_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, (size_t)kControlBytes);
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;

    LinearParams p;
    p.x = a->x;
    p.norm_w = a->norm_weight;
    p.w = a->weight;
    p.residual = a->residual;
    p.out = a->out;
    p.argmax = reinterpret_cast<long long*>(a->argmax);
    p.ctl = static_cast<Control*>(workspace);
    p.ntok = a->batch;
    p.K = K;
    p.N = N;
    p.eps = a->eps;
    // three to eight tokens: tensor-core tiles when the inner dimension splits into 32-wide slices over the eight warps
    p.mma = (options().linear_mma > 0 && a->batch >= options().linear_mma && K % 256 == 0) ? 1 : 0;
    p.rows = kLinStageBytes / (K * 2);
    if (p.mma && p.rows > kLinMmaRows) p.rows = kLinMmaRows;
    p.nchunks = (N + p.rows - 1) / p.rows;
    {
        const int ppt = (K / 8 + kLinConsumerThreads - 1) / kLinConsumerThreads;
        p.lg_ppt = 0;
        while ((1 << p.lg_ppt) < ppt) ++p.lg_ppt;
    }
    size_t off = 0;
    auto take = [&](size_t bytes, size_t align) {
        off = align_up(off, align);
        const size_t at = off;
        off += bytes;
        return (int)at;
    };
    p.off_bars = take(2 * kLinMaxStages * 8, 16);
    const int xtok = p.mma ? kLinMaxTokens : (a->batch > 2 ? (a->batch + 3) / 4 * 4 : a->batch);  // groups of three tokens read a fourth vector
    p.off_red = take(p.mma ? (size_t)2 * kLinConsumerWarps * kLinMmaRows * 8 * 4 : 0, 16);
    p.off_x = take((size_t)xtok * K * 2, 128);
    p.off_ring = take(0, 128);
    const long long room = (long long)dev->max_smem_optin - (long long)off - 1024;
    int nstages = (int)(room / kLinStageBytes);
    if (nstages > kLinMaxStages) nstages = kLinMaxStages;
    if (nstages < 2) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_decode: shapes do not fit in shared memory");
    p.nstages = nstages;
    const size_t smem_bytes = (size_t)p.off_ring + (size_t)nstages * kLinStageBytes;
    const int grid = p.nchunks < dev->sm_count ? p.nchunks : dev->sm_count;

    const void* kernel = (a->dtype == MK36_BF16) ? (const void*)linear_decode_kernel<__nv_bfloat16> : (const void*)linear_decode_kernel<__half>;
    {
        const int rc = ensure_dynamic_smem(kernel, smem_bytes);
        if (rc != MK36_OK) return rc;
    }
    void* params[] = {&p};
    const cudaError_t e = cudaLaunchKernel(kernel, dim3(grid), dim3(kLinThreads), params, smem_bytes, stream);
    if (e != cudaSuccess) MK36_FAIL(MK36_ERR_LAUNCH, "linear_decode: launch failed (grid %d, smem %zu): %s", grid, smem_bytes, cudaGetErrorString(e));
    return MK36_OK;
}

}  // extern "C"
