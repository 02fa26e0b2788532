// Pieces shared by the two split-KV attention kernels: the launch parameters and the in-kernel
// merge of the per-split partials (one bounded grid barrier, then every warp of the grid folds the
// splits of its items with a log-sum-exp combine).
#pragma once

#include "mk36_common.cuh"

namespace mk36 {

struct AttnParams {
    const void* q;
    const void* k;
    const void* v;
    void* out;
    Control* ctl;
    float* part_o;  // [B][Hq][splits][D]
    float* part_m;  // [B][Hq][splits]
    float* part_l;  // [B][Hq][splits]
    int B, Hq, Hkv, D, T;
    int group;      // Hq / Hkv
    int subgroups;  // CTAs that share one KV head's stream because a CTA serves at most GP heads
    int splits;
    float scale;
};

#if defined(__CUDACC__)

constexpr int kAttnMergeMaxSplits = 160;  // splits the one-round-trip merge handles (five per lane)

// The merge proper, after the grid barrier: warp number `first` of `total_warps` takes the items first,
// first + total_warps, ...  An item is (batch, head, 4 channels) when the one-round-trip path applies
// (head_dim a multiple of 4, at most kAttnMergeMaxSplits splits: lanes own the splits, up to five each, so every
// load of the item is issued at once), else (batch, head, 32 channels) with a loop over the splits.
template <typename T>
__device__ __forceinline__ void attention_merge_items(const AttnParams& p, int first, int total_warps, int lane) {
    T* out = static_cast<T*>(p.out);
    if (p.D % 4 == 0 && p.splits <= kAttnMergeMaxSplits) {
        constexpr int kPer = kAttnMergeMaxSplits / 32;
        const int d4 = p.D >> 2;
        const int items = p.B * p.Hq * d4;
        for (int it = first; it < items; it += total_warps) {
            const int bh = it / d4, dc = it - bh * d4;
            const float* pm = p.part_m + (size_t)bh * p.splits;
            const float* pl = p.part_l + (size_t)bh * p.splits;
            const float* po = p.part_o + (size_t)bh * p.splits * p.D + dc * 4;
            float ms[kPer], ls[kPer];
            float4 pa[kPer];
#pragma unroll
            for (int j = 0; j < kPer; ++j) {
                const int sp = lane + 32 * j;
                const bool valid = sp < p.splits;
                ms[j] = valid ? __ldcg(pm + sp) : -INFINITY;
                ls[j] = valid ? __ldcg(pl + sp) : 0.0f;
                pa[j] = valid ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)sp * p.D)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            float mloc = ms[0];
#pragma unroll
            for (int j = 1; j < kPer; ++j) mloc = fmaxf(mloc, ms[j]);
            const float mm = warp_max(mloc);
            float acc[5] = {0.f, 0.f, 0.f, 0.f, 0.f};  // four channels and the normaliser
#pragma unroll
            for (int j = 0; j < kPer; ++j) {
                const float sc = (ms[j] == -INFINITY) ? 0.0f : __expf(ms[j] - mm);
                acc[0] = fmaf(sc, pa[j].x, acc[0]); acc[1] = fmaf(sc, pa[j].y, acc[1]);
                acc[2] = fmaf(sc, pa[j].z, acc[2]); acc[3] = fmaf(sc, pa[j].w, acc[3]);
                acc[4] = fmaf(sc, ls[j], acc[4]);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
#pragma unroll
                for (int i = 0; i < 5; ++i) acc[i] += __shfl_xor_sync(kFullMask, acc[i], off);
            }
            if (lane < 4) {
                const float v = (lane == 0) ? acc[0] : (lane == 1) ? acc[1] : (lane == 2) ? acc[2] : acc[3];
                out[(size_t)bh * p.D + dc * 4 + lane] = from_float<T>(v / acc[4]);
            }
        }
        return;
    }
    const int dchunks = (p.D + 31) / 32;
    const int items = p.B * p.Hq * dchunks;
    for (int it = first; it < items; it += total_warps) {
        const int dc = it % dchunks;
        const int bh = it / dchunks;
        const int d = dc * 32 + lane;
        const float* pm = p.part_m + (size_t)bh * p.splits;
        const float* pl = p.part_l + (size_t)bh * p.splits;
        const float* po = p.part_o + (size_t)bh * p.splits * p.D;
        float mm = -INFINITY;
        for (int s = lane; s < p.splits; s += 32) mm = fmaxf(mm, __ldcg(pm + s));
        mm = warp_max(mm);
        float acc = 0.0f, lsum = 0.0f;
#pragma unroll 4
        for (int s = 0; s < p.splits; ++s) {
            const float ms = __ldcg(pm + s);
            const float sc = (ms == -INFINITY) ? 0.0f : expf(ms - mm);
            lsum = fmaf(sc, __ldcg(pl + s), lsum);
            if (d < p.D) acc = fmaf(sc, __ldcg(po + (size_t)s * p.D + d), acc);
        }
        if (d < p.D) out[(size_t)bh * p.D + d] = from_float<T>(acc / lsum);
    }
}

// Every thread of every CTA calls this after its CTA has written its partials.  Returns false when
// the barrier wait ran out (the status word then holds the code).
template <typename T>
__device__ __forceinline__ bool attention_merge_partials(const AttnParams& p, int warps_per_cta, int* s_flag) {
    if (!grid_barrier(p.ctl, gridDim.x, 0, kStatusAttnBarrier, s_flag)) return false;
    if (threadIdx.x == 0) barrier_finish(p.ctl, gridDim.x);
    attention_merge_items<T>(p, blockIdx.x * warps_per_cta + (threadIdx.x >> 5), gridDim.x * warps_per_cta, threadIdx.x & 31);
    return true;
}

#endif

}  // namespace mk36
