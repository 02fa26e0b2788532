// Full-attention GQA decode, tensor-core variant for sm_100a (bf16 / f16, head_dim 64/128/256,
// up to 8 query heads per KV head).
//
// A CTA owns (batch, kv head, token range); its eight warps take 16-token tiles round-robin.  The
// query heads that share the KV head are the N side of mma.sync.m16n8k16, so K and V are read
// once for the whole GQA group (the reference streams them once per query head and reads K twice,
// csrc/attention_decode.cu:33-106):
//     S[16 tokens, 8 heads] = K_tile[16, D] . Q^T[D, 8]            (M = tokens, K = channels)
//     O^T[D, 8 heads]      += V_tile^T[D, 16] . P^T[16 tokens, 8]  (M = channels, K = tokens)
// K and V fragments come straight from global memory with 128-bit loads, no shared-memory staging
// and no ldmatrix: for S the contraction index is permuted identically on both operands (lane
// (g,t) takes channels 8t..8t+7 of each 32-wide slice of rows g and g+8); for P.V each lane owns a
// contiguous run of D/8 channels of its four tokens (2t, 2t+1, 2t+8, 2t+9) and pairs them up with
// byte permutes, and P reaches the operand layout with one 8x8 transpose (movmatrix) per half tile.
// The loads of the next tile are issued before the math of the current one (K after the score
// MMAs have consumed it, V after the output MMAs), so each warp keeps 16 KB in flight.
//
// Online soft-max state is per warp; warps are folded in shared memory, splits through the shared
// merge (one bounded grid barrier).  Arithmetic follows mega_kernel_qwen36/reference.py:117-145
// (fp32 scores and accumulation); the probabilities enter the second product rounded to the
// storage dtype and the normaliser is summed from the same rounded values.
#include <cfloat>

#include "mk36_attention.cuh"

namespace mk36 {

constexpr int kMmaAttnThreads = 256;
constexpr int kMmaAttnWarps = kMmaAttnThreads / 32;
constexpr int kTileTokens = 16;

template <typename T>
__device__ __forceinline__ void mma16816(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0, unsigned b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                                        unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&d)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3, unsigned b0,
                                                 unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ unsigned pack2(float lo, float hi);
template <>
__device__ __forceinline__ unsigned pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}
template <>
__device__ __forceinline__ unsigned pack2<__half>(float lo, float hi) {
    __half2 v = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

template <typename T>
__device__ __forceinline__ float2 unpack2(unsigned v);
template <>
__device__ __forceinline__ float2 unpack2<__nv_bfloat16>(unsigned v) {
    return make_float2(__uint_as_float(v << 16), __uint_as_float(v & 0xffff0000u));
}
template <>
__device__ __forceinline__ float2 unpack2<__half>(unsigned v) {
    return __half22float2(*reinterpret_cast<const __half2*>(&v));
}

__device__ __forceinline__ unsigned transpose8x8(unsigned v) {
    unsigned r;
    asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(r) : "r"(v));
    return r;
}

template <typename T, int D>
__global__ void __launch_bounds__(kMmaAttnThreads, 1) attention_decode_mma_kernel(const AttnParams p) {
    constexpr int NSL = D / 32;   // 32-wide channel slices of the score product
    constexpr int NW = D / 16;    // 32-bit words of V per lane and token = M tiles of the output product
    constexpr int NV4 = D / 64;   // 128-bit loads of V per lane and token
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ float s_fold_m[8];
    T* sq = reinterpret_cast<T*>(smem);                               // [8][D] query heads of the group (zero padded)
    float* s_o = reinterpret_cast<float*>(smem + 8 * D * sizeof(T));  // [warps][8][D]
    float* s_m = s_o + kMmaAttnWarps * 8 * D;                          // [warps][8]
    float* s_l = s_m + kMmaAttnWarps * 8;                              // [warps][8]

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;

    int item = blockIdx.x;
    const int split = item % p.splits;
    item /= p.splits;
    const int kvh = item % p.Hkv;
    const int b = item / p.Hkv;
    const int hq0 = kvh * p.group;

    const bool tracer = (blockIdx.x == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);

    // token range of this CTA in whole tiles; warps take tiles round-robin
    const int tiles_total = (p.T + kTileTokens - 1) / kTileTokens;
    const int tile_begin = (int)(((long long)tiles_total * split) / p.splits);
    const int tile_end = (int)(((long long)tiles_total * (split + 1)) / p.splits);

    const size_t tok_stride = (size_t)p.Hkv * D;  // elements between consecutive tokens
    const T* kbase = static_cast<const T*>(p.k) + (size_t)b * p.T * tok_stride + (size_t)kvh * D;
    const T* vbase = static_cast<const T*>(p.v) + (size_t)b * p.T * tok_stride + (size_t)kvh * D;

    float o[NW][4];
#pragma unroll
    for (int m = 0; m < NW; ++m) { o[m][0] = 0.f; o[m][1] = 0.f; o[m][2] = 0.f; o[m][3] = 0.f; }
    float mrun[2] = {-INFINITY, -INFINITY};  // running max of heads 2t, 2t+1
    float lrun[2] = {0.0f, 0.0f};            // this lane's share of the running sums

    uint4 kreg[2][NSL];   // K: rows g and g+8, channels 32*sl + 8t ..
    uint4 vreg[4][NV4];   // V: tokens 2t, 2t+1, 2t+8, 2t+9, channels g*D/8 ..
    const uint4 zero4 = make_uint4(0, 0, 0, 0);

    auto load_k = [&](int tile) {
        const int tok0 = tile * kTileTokens;
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            const int tok = tok0 + g + 8 * r;
            const T* row = kbase + (size_t)tok * tok_stride + 8 * t;
#pragma unroll
            for (int sl = 0; sl < NSL; ++sl) kreg[r][sl] = (tok < p.T) ? ld_stream_u4(row + 32 * sl) : zero4;
        }
    };
    auto load_v = [&](int tile) {
        const int tok0 = tile * kTileTokens;
#pragma unroll
        for (int r = 0; r < 4; ++r) {
            const int tok = tok0 + 2 * t + (r & 1) + ((r & 2) ? 8 : 0);
            const T* row = vbase + (size_t)tok * tok_stride + g * (D / 8);
#pragma unroll
            for (int j = 0; j < NV4; ++j) vreg[r][j] = (tok < p.T) ? ld_stream_u4(row + 8 * j) : zero4;
        }
    };

    int tile = tile_begin + warp;
    if (tile < tile_end) {
        load_k(tile);
        load_v(tile);
    }
    // the query heads of the group, zero padded to 8 rows (one 16-byte load per thread and pass)
    {
        const T* q = static_cast<const T*>(p.q) + ((size_t)b * p.Hq + hq0) * D;
        for (int i = tid * 8; i < 8 * D; i += kMmaAttnThreads * 8) {
            const int h = i / D;
            *reinterpret_cast<uint4*>(sq + i) = (h < p.group) ? *reinterpret_cast<const uint4*>(q + i) : make_uint4(0, 0, 0, 0);
        }
    }
    __syncthreads();
    if (tracer) trace_stamp(p.ctl, 1);
    bool first_tile = true;
    for (; tile < tile_end; tile += kMmaAttnWarps) {
        const int tok0 = tile * kTileTokens;
        // ---- scores: two accumulators to shorten the dependent MMA chain ----
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int sl = 0; sl < NSL; ++sl) {
            const uint4 qv = *reinterpret_cast<const uint4*>(sq + (size_t)g * D + 32 * sl + 8 * t);
            mma16816<T>(s0, kreg[0][sl].x, kreg[1][sl].x, kreg[0][sl].y, kreg[1][sl].y, qv.x, qv.y);
            mma16816<T>(s1, kreg[0][sl].z, kreg[1][sl].z, kreg[0][sl].w, kreg[1][sl].w, qv.z, qv.w);
        }
        const int next = tile + kMmaAttnWarps;
        if (next < tile_end) load_k(next);  // K registers are free again

        float s[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) s[i] = (s0[i] + s1[i]) * p.scale;
        if (tok0 + g >= p.T) { s[0] = -INFINITY; s[1] = -INFINITY; }
        if (tok0 + g + 8 >= p.T) { s[2] = -INFINITY; s[3] = -INFINITY; }

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
        // The probabilities enter the second product rounded to the storage dtype; the normaliser is summed
        // from the same rounded values, so that the output weights still add up to one (with the unrounded
        // sum a short context, where nothing averages out, would carry the rounding error of each weight).
        const unsigned pk01 = pack2<T>(p0, p1), pk23 = pack2<T>(p2, p3);
        const float2 r01 = unpack2<T>(pk01), r23 = unpack2<T>(pk23);
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
        // probabilities as the B operand: (tokens 2t,2t+1 | 2t+8,2t+9 ; head g)
        const unsigned b0 = transpose8x8(pk01);
        const unsigned b1 = transpose8x8(pk23);

        // ---- output: word m of a token holds channels g*D/8 + 2m, 2m+1 ----
#pragma unroll
        for (int m = 0; m < NW; ++m) {
            const unsigned w0 = reinterpret_cast<const unsigned*>(&vreg[0][m / 4])[m % 4];
            const unsigned w1 = reinterpret_cast<const unsigned*>(&vreg[1][m / 4])[m % 4];
            const unsigned w2 = reinterpret_cast<const unsigned*>(&vreg[2][m / 4])[m % 4];
            const unsigned w3 = reinterpret_cast<const unsigned*>(&vreg[3][m / 4])[m % 4];
            mma16816<T>(o[m], __byte_perm(w0, w1, 0x5410), __byte_perm(w0, w1, 0x7632), __byte_perm(w2, w3, 0x5410),
                        __byte_perm(w2, w3, 0x7632), b0, b1);
        }
        if (next < tile_end) load_v(next);  // V registers are free again
        if (tracer && first_tile) trace_stamp(p.ctl, 2);
        first_tile = false;
    }
    if (tracer) trace_stamp(p.ctl, 3);
    // sums over the eight lanes that share a head pair
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
        lrun[0] += __shfl_xor_sync(kFullMask, lrun[0], off);
        lrun[1] += __shfl_xor_sync(kFullMask, lrun[1], off);
    }

    // ---- fold the warps: o[m] = {(ch lo, head 2t), (ch lo, head 2t+1), (ch hi, head 2t), (ch hi, head 2t+1)} ----
    float* wo = s_o + (size_t)warp * 8 * D;
#pragma unroll
    for (int m = 0; m < NW; ++m) {
        const int ch = g * (D / 8) + 2 * m;
        wo[(2 * t) * D + ch] = o[m][0];
        wo[(2 * t + 1) * D + ch] = o[m][1];
        wo[(2 * t) * D + ch + 1] = o[m][2];
        wo[(2 * t + 1) * D + ch + 1] = o[m][3];
    }
    if (g == 0) {
        s_m[warp * 8 + 2 * t] = mrun[0];
        s_m[warp * 8 + 2 * t + 1] = mrun[1];
        s_l[warp * 8 + 2 * t] = lrun[0];
        s_l[warp * 8 + 2 * t + 1] = lrun[1];
    }
    __syncthreads();
    if (tracer) trace_stamp(p.ctl, 4);
    if (tid == 0) cta_stamp(p.ctl, blockIdx.x, 0);
    // per (warp, head) rescale factors, once; s_l is reused for them
    float f_sc = 0.0f, f_lw = 0.0f, f_mm = 0.0f;
    if (tid < 8 * kMmaAttnWarps) {
        const int h = tid & 7;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kMmaAttnWarps; ++w) mm = fmaxf(mm, s_m[w * 8 + h]);
        const float mw = s_m[tid];
        f_sc = (mw == -INFINITY) ? 0.0f : __expf(mw - mm);
        f_lw = s_l[tid] * f_sc;
        f_mm = mm;
    }
    __syncthreads();
    if (tid < 8 * kMmaAttnWarps) {
        s_l[tid] = f_lw;  // scaled share of the sum
        s_m[tid] = f_sc;  // factor for the outputs
        if (tid < 8) s_fold_m[tid] = f_mm;
    }
    __syncthreads();
    for (int idx = tid; idx < p.group * D; idx += kMmaAttnThreads) {
        const int h = idx / D, d = idx - h * D;
        float acc = 0.0f;
#pragma unroll
        for (int w = 0; w < kMmaAttnWarps; ++w) acc = fmaf(s_m[w * 8 + h], s_o[((size_t)w * 8 + h) * D + d], acc);
        const size_t pi = ((size_t)b * p.Hq + hq0 + h) * p.splits + split;
        p.part_o[pi * D + d] = acc;
        if (d == 0) {
            float lsum = 0.0f;
#pragma unroll
            for (int w = 0; w < kMmaAttnWarps; ++w) lsum += s_l[w * 8 + h];
            p.part_m[pi] = s_fold_m[h];
            p.part_l[pi] = lsum;
        }
    }
    if (tracer) trace_stamp(p.ctl, 5);
    attention_merge_partials<T>(p, kMmaAttnWarps, &s_flag);
    if (tracer) trace_stamp(p.ctl, 6);
}

namespace {

template <typename T>
const void* mma_kernel_for(int d) {
    switch (d) {
        case 64: return (const void*)attention_decode_mma_kernel<T, 64>;
        case 128: return (const void*)attention_decode_mma_kernel<T, 128>;
        case 256: return (const void*)attention_decode_mma_kernel<T, 256>;
        default: return nullptr;
    }
}

}  // namespace

// Launches the tensor-core variant when the shapes suit it and sets *handled; otherwise leaves
// *handled false (no error) and the caller uses the general kernel.
int attention_decode_mma_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    const int D = a->head_dim, group = a->query_heads / a->kv_heads;
    if (group > 8 || (D != 64 && D != 128 && D != 256)) return MK36_OK;
    const void* ptrs[] = {a->q, a->k_cache, a->v_cache};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const void* kernel = (a->dtype == MK36_BF16) ? mma_kernel_for<__nv_bfloat16>(D) : mma_kernel_for<__half>(D);
    if (!kernel) return MK36_OK;
    const size_t smem = (size_t)8 * D * 2 + ((size_t)kMmaAttnWarps * 8 * D + 2 * kMmaAttnWarps * 8) * 4;
    {
        const int rc_smem = ensure_dynamic_smem(kernel, smem);
        if (rc_smem != MK36_OK) return rc_smem;
    }
    const long long max_ctas = dev->sm_count;  // one CTA per SM (register budget)
    const long long per_batch = a->kv_heads;
    if (per_batch > max_ctas) return MK36_OK;
    int batch_per_launch = (int)(max_ctas / per_batch);
    if (batch_per_launch > a->batch) batch_per_launch = a->batch;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "full_attention_decode: workspace is NULL or not 256-byte aligned");

    const size_t es = 2;
    auto splits_for = [&](int nb) {
        long long splits = max_ctas / ((long long)nb * a->kv_heads);
        const long long by_len = (a->seq_len + 8 * kTileTokens - 1) / (8 * kTileTokens);  // at least one tile per warp
        if (splits > by_len) splits = by_len;
        return splits < 1 ? 1ll : splits;
    };
    auto scratch_for = [&](int nb, long long splits) {
        const size_t heads = (size_t)nb * a->query_heads;
        return align_up(heads * splits * D * 4, 256) + 2 * align_up(heads * splits * 4, 256);
    };
    // every launch of the call must fit before the first one is made: a refused call writes nothing
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        const int nb = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        const size_t scratch = scratch_for(nb, splits_for(nb));
        if (workspace_bytes < kControlBytes + scratch)
            MK36_FAIL(MK36_ERR_WORKSPACE, "full_attention_decode: workspace too small (%zu < %zu bytes)", workspace_bytes,
                      kControlBytes + scratch);
    }
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        const int nb = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        const long long splits = splits_for(nb);
        const size_t heads = (size_t)nb * a->query_heads;
        AttnParams p;
        p.q = static_cast<const unsigned char*>(a->q) + (size_t)b0 * a->query_heads * D * es;
        p.k = static_cast<const unsigned char*>(a->k_cache) + (size_t)b0 * a->seq_len * a->kv_heads * D * es;
        p.v = static_cast<const unsigned char*>(a->v_cache) + (size_t)b0 * a->seq_len * a->kv_heads * D * es;
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
        p.Hkv = a->kv_heads;
        p.D = D;
        p.T = a->seq_len;
        p.group = group;
        p.subgroups = 1;
        p.splits = (int)splits;
        p.scale = a->scale;
        const unsigned grid = (unsigned)((long long)nb * a->kv_heads * splits);
        void* params[] = {&p};
        int rc = launch_cooperative(kernel, dim3(grid), dim3(kMmaAttnThreads), smem, stream, params, "full_attention_decode(mma)");
        if (rc != MK36_OK) return rc;
    }
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
