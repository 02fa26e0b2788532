// Pieces shared by the two split-KV attention kernels: the launch parameters and the in-kernel
// merge of the per-split partials (one bounded grid barrier, then every warp of the grid folds the
// splits of one (batch, head, 32 channels) item with a log-sum-exp combine).
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

// Every thread of every CTA calls this after its CTA has written its partials.  Returns false when
// the barrier wait ran out (the status word then holds the code).
template <typename T>
__device__ __forceinline__ bool attention_merge_partials(const AttnParams& p, int warps_per_cta, int* s_flag) {
    if (!grid_barrier(p.ctl, gridDim.x, 0, kStatusAttnBarrier, s_flag)) return false;
    if (threadIdx.x == 0) barrier_finish(p.ctl, gridDim.x);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int total_warps = gridDim.x * warps_per_cta;
    T* out = static_cast<T*>(p.out);
    if (p.D % 8 == 0 && p.splits <= 128) {
        // One warp per (batch, head, 8 channels): lanes own the splits (up to four each), so every
        // load of the item is issued at once and the merge costs one memory round trip.
        const int d8 = p.D >> 3;
        const int items = p.B * p.Hq * d8;
        for (int it = blockIdx.x * warps_per_cta + warp; it < items; it += total_warps) {
            const int bh = it / d8, dc = it - bh * d8;
            const float* pm = p.part_m + (size_t)bh * p.splits;
            const float* pl = p.part_l + (size_t)bh * p.splits;
            const float* po = p.part_o + (size_t)bh * p.splits * p.D + dc * 8;
            float ms[4], ls[4];
            float4 pa[4], pb[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int sp = lane + 32 * j;
                const bool valid = sp < p.splits;
                ms[j] = valid ? __ldcg(pm + sp) : -INFINITY;
                ls[j] = valid ? __ldcg(pl + sp) : 0.0f;
                pa[j] = valid ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)sp * p.D)) : make_float4(0.f, 0.f, 0.f, 0.f);
                pb[j] = valid ? __ldcg(reinterpret_cast<const float4*>(po + (size_t)sp * p.D + 4)) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
            const float mm = warp_max(fmaxf(fmaxf(ms[0], ms[1]), fmaxf(ms[2], ms[3])));
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            float lsum = 0.0f;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float sc = (ms[j] == -INFINITY) ? 0.0f : expf(ms[j] - mm);
                lsum = fmaf(sc, ls[j], lsum);
                acc[0] = fmaf(sc, pa[j].x, acc[0]); acc[1] = fmaf(sc, pa[j].y, acc[1]);
                acc[2] = fmaf(sc, pa[j].z, acc[2]); acc[3] = fmaf(sc, pa[j].w, acc[3]);
                acc[4] = fmaf(sc, pb[j].x, acc[4]); acc[5] = fmaf(sc, pb[j].y, acc[5]);
                acc[6] = fmaf(sc, pb[j].z, acc[6]); acc[7] = fmaf(sc, pb[j].w, acc[7]);
            }
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) {
                lsum += __shfl_xor_sync(kFullMask, lsum, off);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(kFullMask, acc[i], off);
            }
            if (lane < 8) {
                float v = acc[0];
#pragma unroll
                for (int i = 1; i < 8; ++i)
                    if (lane == i) v = acc[i];
                out[(size_t)bh * p.D + dc * 8 + lane] = from_float<T>(v / lsum);
            }
        }
        return true;
    }
    const int dchunks = (p.D + 31) / 32;
    const int items = p.B * p.Hq * dchunks;
    for (int it = blockIdx.x * warps_per_cta + warp; it < items; it += total_warps) {
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
    return true;
}

#endif

}  // namespace mk36
