// Full-attention GQA decode of one query token for sm_100a: split-KV with an in-kernel combine.
//
// One cooperative launch.  The cache is cut along the token axis into `splits` contiguous
// ranges; a CTA owns (batch, kv head, head sub-group, split), streams its K and V rows once for
// all query heads of the group (the reference re-reads them once per query head and reads K
// twice: csrc/attention_decode.cu:33-106), keeps an online soft-max per warp, folds the warps in
// shared memory and writes one partial (max, sum, unnormalised output) per head.  After one
// bounded grid barrier the partials are merged by all CTAs in parallel (the reference merges in
// a second launch with one serial thread per head: csrc/attention_decode.cu:108-148).
//
// Arithmetic follows mega_kernel_qwen36/reference.py:117-145: fp32 scores, fp32 soft-max over
// the whole cache, fp32 accumulation, one rounding to the output dtype.
#include <cfloat>

#include "mk36_attention.cuh"

namespace mk36 {

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kMaxHeadDim = 256;
constexpr int kDimPerLane = kMaxHeadDim / 32;

// Generic path: any dtype, any head_dim <= 256, CUDA cores.  Lane l owns channels l, l+32, ...
template <typename T, int GP>
__global__ void __launch_bounds__(kAttnThreads) attention_decode_generic_kernel(const AttnParams p) {
    __shared__ float s_o[kAttnWarps][GP][kMaxHeadDim];
    __shared__ float s_m[kAttnWarps][GP];
    __shared__ float s_l[kAttnWarps][GP];
    __shared__ int s_flag;

    const int lane = threadIdx.x & 31;
    const int warp = threadIdx.x >> 5;

    // ---- decode the CTA's work item ----
    int item = blockIdx.x;
    const int split = item % p.splits;
    item /= p.splits;
    const int sub = item % p.subgroups;
    item /= p.subgroups;
    const int kvh = item % p.Hkv;
    const int b = item / p.Hkv;
    const int g0 = sub * GP;                                  // first head of the sub-group inside the GQA group
    const int gcount = (p.group - g0 < GP) ? (p.group - g0) : GP;
    const int hq0 = kvh * p.group + g0;

    const int t_begin = (int)(((long long)p.T * split) / p.splits);
    const int t_end = (int)(((long long)p.T * (split + 1)) / p.splits);

    const T* q = static_cast<const T*>(p.q);
    const T* kc = static_cast<const T*>(p.k);
    const T* vc = static_cast<const T*>(p.v);

    float qf[GP][kDimPerLane];
    float of[GP][kDimPerLane];
    float m[GP], l[GP];
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.0f;
#pragma unroll
        for (int j = 0; j < kDimPerLane; ++j) {
            const int d = lane + 32 * j;
            qf[g][j] = (g < gcount && d < p.D) ? to_float<T>(q[((size_t)b * p.Hq + hq0 + g) * p.D + d]) * p.scale : 0.0f;
            of[g][j] = 0.0f;
        }
    }

    const size_t tok_stride = (size_t)p.Hkv * p.D;
    const size_t base = (size_t)b * p.T * tok_stride + (size_t)kvh * p.D;
    for (int t = t_begin + warp; t < t_end; t += kAttnWarps) {
        const T* kr = kc + base + (size_t)t * tok_stride;
        const T* vr = vc + base + (size_t)t * tok_stride;
        float kf[kDimPerLane], vf[kDimPerLane];
#pragma unroll
        for (int j = 0; j < kDimPerLane; ++j) {
            const int d = lane + 32 * j;
            kf[j] = (d < p.D) ? to_float<T>(kr[d]) : 0.0f;
            vf[j] = (d < p.D) ? to_float<T>(vr[d]) : 0.0f;
        }
#pragma unroll
        for (int g = 0; g < GP; ++g) {
            float s = 0.0f;
#pragma unroll
            for (int j = 0; j < kDimPerLane; ++j) s = fmaf(qf[g][j], kf[j], s);
            s = warp_sum(s);
            if (s > m[g]) {  // warp-uniform
                const float corr = expf(m[g] - s);
                l[g] *= corr;
#pragma unroll
                for (int j = 0; j < kDimPerLane; ++j) of[g][j] *= corr;
                m[g] = s;
            }
            const float pw = expf(s - m[g]);
            l[g] += pw;
#pragma unroll
            for (int j = 0; j < kDimPerLane; ++j) of[g][j] = fmaf(pw, vf[j], of[g][j]);
        }
    }

    // ---- fold the warps of this CTA ----
#pragma unroll
    for (int g = 0; g < GP; ++g) {
        if (lane == 0) {
            s_m[warp][g] = m[g];
            s_l[warp][g] = l[g];
        }
#pragma unroll
        for (int j = 0; j < kDimPerLane; ++j) s_o[warp][g][lane + 32 * j] = of[g][j];
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < gcount * p.D; idx += kAttnThreads) {
        const int g = idx / p.D, d = idx % p.D;
        float mm = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) mm = fmaxf(mm, s_m[w][g]);
        float acc = 0.0f, lsum = 0.0f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float sc = (s_m[w][g] == -INFINITY) ? 0.0f : expf(s_m[w][g] - mm);
            acc = fmaf(sc, s_o[w][g][d], acc);
            lsum = fmaf(sc, s_l[w][g], lsum);
        }
        const size_t pi = ((size_t)b * p.Hq + hq0 + g) * p.splits + split;
        p.part_o[pi * p.D + d] = acc;
        if (d == 0) {
            p.part_m[pi] = mm;
            p.part_l[pi] = lsum;
        }
    }

    // ---- one grid barrier, then every CTA merges a share of the outputs ----
    attention_merge_partials<T>(p, kAttnWarps, &s_flag);
}

// -------------------------------------------------------------------------------------------
// Host side
// -------------------------------------------------------------------------------------------
namespace {

struct AttnPlan {
    int gp;         // heads per CTA
    int subgroups;
    int splits;
    size_t scratch_bytes;
};

template <typename T>
const void* generic_kernel_for(int gp) {
    switch (gp) {
        case 1: return (const void*)attention_decode_generic_kernel<T, 1>;
        case 2: return (const void*)attention_decode_generic_kernel<T, 2>;
        default: return (const void*)attention_decode_generic_kernel<T, 4>;
    }
}

const void* generic_kernel(int dtype, int gp) {
    if (dtype == MK36_BF16) return generic_kernel_for<__nv_bfloat16>(gp);
    if (dtype == MK36_F16) return generic_kernel_for<__half>(gp);
    return generic_kernel_for<float>(gp);
}

int check_attention_args(const mk36_attention_args* a) {
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "full_attention_decode: args is NULL");
    if (!a->q || !a->k_cache || !a->v_cache || !a->out) MK36_FAIL(MK36_ERR_INVALID_ARG, "full_attention_decode: NULL tensor pointer");
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16 && a->dtype != MK36_F32)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "full_attention_decode: unsupported dtype %d", a->dtype);
    if (a->batch <= 0 || a->query_heads <= 0 || a->kv_heads <= 0 || a->head_dim <= 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "full_attention_decode: sizes must be positive");
    if (a->query_heads % a->kv_heads != 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "query_heads must be divisible by kv_heads");
    if (a->head_dim > kMaxHeadDim) MK36_FAIL(MK36_ERR_UNSUPPORTED, "head_dim > 256 is not supported by this kernel");
    if (a->seq_len <= 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "seq_len must be positive");
    return MK36_OK;
}

void plan_generic(const mk36_attention_args& a, int max_ctas, AttnPlan* plan) {
    const int group = a.query_heads / a.kv_heads;
    int gp = 1;
    while (gp < group && gp < 4) gp <<= 1;
    plan->gp = gp;
    plan->subgroups = (group + gp - 1) / gp;
    const long long base = (long long)a.batch * a.kv_heads * plan->subgroups;
    long long splits = max_ctas / base;
    const long long by_len = (a.seq_len + 31) / 32;  // at least 32 tokens per split
    if (splits > by_len) splits = by_len;
    if (splits < 1) splits = 1;
    plan->splits = (int)splits;
    const size_t heads = (size_t)a.batch * a.query_heads;
    plan->scratch_bytes = align_up(heads * plan->splits * a.head_dim * 4, 256) + 2 * align_up(heads * plan->splits * 4, 256);
}

}  // namespace

int attention_decode_mma_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool* handled);
int attention_decode_stream_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream, bool* handled);

int attention_decode_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream) {
    int rc = check_attention_args(a);
    if (rc != MK36_OK) return rc;
    if (!options().force_generic) {
        bool handled = false;
        if (options().attn_stream) {
            rc = attention_decode_stream_launch(a, workspace, workspace_bytes, stream, &handled);
            if (rc != MK36_OK || handled) return rc;
        }
        rc = attention_decode_mma_launch(a, workspace, workspace_bytes, stream, &handled);
        if (rc != MK36_OK || handled) return rc;
    }
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "full_attention_decode: workspace is NULL or not 256-byte aligned");

    const int group = a->query_heads / a->kv_heads;
    int gp = 1;
    while (gp < group && gp < 4) gp <<= 1;
    const void* kernel = generic_kernel(a->dtype, gp);
    static thread_local const void* cached_kernel = nullptr;
    static thread_local int cached_occ = 0;
    if (cached_kernel != kernel) {
        cached_occ = max_ctas_per_sm(kernel, kAttnThreads, 0);
        if (cached_occ <= 0) MK36_FAIL(MK36_ERR_LAUNCH, "full_attention_decode: kernel does not fit on an SM");
        cached_kernel = kernel;
    }
    // when one (batch, kv head, sub-group) set alone exceeds the co-resident limit, run it in rounds
    const int subgroups = (group + gp - 1) / gp;
    const long long per_batch = (long long)a->kv_heads * subgroups;
    const long long max_ctas = (long long)dev->sm_count * cached_occ;
    if (per_batch > max_ctas) MK36_FAIL(MK36_ERR_UNSUPPORTED, "full_attention_decode: too many heads for one launch");
    int batch_per_launch = (int)(max_ctas / per_batch);
    if (batch_per_launch > a->batch) batch_per_launch = a->batch;

    const size_t es = a->dtype == MK36_F32 ? 4 : 2;
    // every launch of the call must fit before the first one is made: a refused call writes nothing
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        mk36_attention_args sub = *a;
        sub.batch = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        AttnPlan plan;
        plan_generic(sub, (int)max_ctas, &plan);
        if (workspace_bytes < kControlBytes + plan.scratch_bytes)
            MK36_FAIL(MK36_ERR_WORKSPACE, "full_attention_decode: workspace too small (%zu < %zu bytes)", workspace_bytes,
                      kControlBytes + plan.scratch_bytes);
    }
    for (int b0 = 0; b0 < a->batch; b0 += batch_per_launch) {
        mk36_attention_args sub = *a;
        sub.batch = (a->batch - b0 < batch_per_launch) ? (a->batch - b0) : batch_per_launch;
        AttnPlan plan;
        plan_generic(sub, (int)max_ctas, &plan);
        AttnParams p;
        p.q = static_cast<const unsigned char*>(a->q) + (size_t)b0 * a->query_heads * a->head_dim * es;
        p.k = static_cast<const unsigned char*>(a->k_cache) + (size_t)b0 * a->seq_len * a->kv_heads * a->head_dim * es;
        p.v = static_cast<const unsigned char*>(a->v_cache) + (size_t)b0 * a->seq_len * a->kv_heads * a->head_dim * es;
        p.out = static_cast<unsigned char*>(a->out) + (size_t)b0 * a->query_heads * a->head_dim * es;
        p.ctl = static_cast<Control*>(workspace);
        unsigned char* scratch = static_cast<unsigned char*>(workspace) + kControlBytes;
        const size_t heads = (size_t)sub.batch * a->query_heads;
        p.part_o = reinterpret_cast<float*>(scratch);
        scratch += align_up(heads * plan.splits * a->head_dim * 4, 256);
        p.part_m = reinterpret_cast<float*>(scratch);
        scratch += align_up(heads * plan.splits * 4, 256);
        p.part_l = reinterpret_cast<float*>(scratch);
        p.B = sub.batch;
        p.Hq = a->query_heads;
        p.Hkv = a->kv_heads;
        p.D = a->head_dim;
        p.T = a->seq_len;
        p.group = group;
        p.subgroups = plan.subgroups;
        p.splits = plan.splits;
        p.scale = a->scale;
        const unsigned grid = (unsigned)((long long)sub.batch * a->kv_heads * plan.subgroups * plan.splits);
        void* params[] = {&p};
        rc = launch_cooperative(kernel, dim3(grid), dim3(kAttnThreads), 0, stream, params, "full_attention_decode");
        if (rc != MK36_OK) return rc;
    }
    return MK36_OK;
}

}  // namespace mk36

using namespace mk36;

extern "C" {

size_t mk36_attention_workspace_bytes(const mk36_attention_args* a) {
    if (!a || a->batch <= 0 || a->query_heads <= 0 || a->head_dim <= 0) return 0;
    // A launch holds at most (co-resident CTAs) x (heads per CTA) partial rows; 148 SMs x 8 CTAs
    // x 8 heads bounds that on any sm_100 part.
    const size_t rows = (size_t)148 * 8 * 8;
    return kControlBytes + align_up(rows * a->head_dim * 4, 256) + 2 * align_up(rows * 4, 256);
}

int mk36_full_attention_decode(const mk36_attention_args* args, void* workspace, size_t workspace_bytes, void* stream) {
    return attention_decode_launch(args, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
