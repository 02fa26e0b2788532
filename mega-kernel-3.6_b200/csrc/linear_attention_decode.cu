// Linear-attention recurrent decode step for sm_100a.
//
//   S'[kd, vd] = decay * S[kd, vd] + k[kd] * (beta * v[vd])        (fp32 state)
//   out[vd]    = sum_kd q[kd] * S'[kd, vd]
//
// One CTA owns a slice of 32 value columns of one (batch, value head) state matrix, so at batch
// 1 with 32 heads x 128 columns there are 128 CTAs (the reference's kernel, a thread per output
// column with a serial loop over kd, runs 16: csrc/linear_attention_decode.cu:10-42, 77).
// The state update uses separately rounded multiply / add (no FMA contraction) so that the new
// state is bit-identical to reference.py:164 (`state.mul(decay) + einsum(k, v)`).
#include "mk36_common.cuh"

namespace mk36 {

constexpr int kLinThreads = 256;
constexpr int kLinCols = 32;

struct LinParams {
    const void* q;
    const void* k;
    const void* v;
    const float* state;
    void* out;
    float* new_state;
    const float* decay_ph;
    const float* beta_ph;
    int B, Hk, Hv, Dk, Dv;
    float decay;
};

template <typename T, int VEC>
__global__ void __launch_bounds__(kLinThreads) linear_attention_kernel(const LinParams p) {
    constexpr int CT = kLinCols / VEC;     // threads across the column slice
    constexpr int RG = kLinThreads / CT;   // row groups
    extern __shared__ float s_dyn[];       // q[Dk], k[Dk]
    __shared__ float s_red[RG][kLinCols + 1];

    const int slices = (p.Dv + kLinCols - 1) / kLinCols;
    const int slice = blockIdx.x % slices;
    const int bh = blockIdx.x / slices;
    const int h = bh % p.Hv;
    const int b = bh / p.Hv;
    const int hk = h / (p.Hv / p.Hk);

    float* s_q = s_dyn;
    float* s_k = s_dyn + p.Dk;
    const T* q = static_cast<const T*>(p.q) + ((size_t)b * p.Hk + hk) * p.Dk;
    const T* k = static_cast<const T*>(p.k) + ((size_t)b * p.Hk + hk) * p.Dk;
    for (int i = threadIdx.x; i < p.Dk; i += kLinThreads) {
        s_q[i] = to_float<T>(q[i]);
        s_k[i] = to_float<T>(k[i]);
    }

    const int ct = threadIdx.x % CT;
    const int rg = threadIdx.x / CT;
    const int col0 = slice * kLinCols + ct * VEC;
    const float decay = p.decay_ph ? p.decay_ph[(size_t)b * p.Hv + h] : p.decay;
    const float beta = p.beta_ph ? p.beta_ph[(size_t)b * p.Hv + h] : 1.0f;
    const T* v = static_cast<const T*>(p.v) + ((size_t)b * p.Hv + h) * p.Dv;

    float vv[VEC], o[VEC];
#pragma unroll
    for (int j = 0; j < VEC; ++j) {
        const float raw = (col0 + j < p.Dv) ? to_float<T>(v[col0 + j]) : 0.0f;
        vv[j] = p.beta_ph ? __fmul_rn(raw, beta) : raw;
        o[j] = 0.0f;
    }
    __syncthreads();

    const size_t base = ((size_t)b * p.Hv + h) * p.Dk * p.Dv;
    const float* src = p.state + base;
    float* dst = p.new_state + base;

    if (VEC == 4) {
        if (col0 < p.Dv) {  // Dv % 4 == 0 on this path, so the whole float4 is in range
#pragma unroll 4
            for (int kd = rg; kd < p.Dk; kd += RG) {
                const float4 s = *reinterpret_cast<const float4*>(src + (size_t)kd * p.Dv + col0);
                const float kk = s_k[kd], qq = s_q[kd];
                float4 n;
                n.x = __fadd_rn(__fmul_rn(s.x, decay), __fmul_rn(kk, vv[0]));
                n.y = __fadd_rn(__fmul_rn(s.y, decay), __fmul_rn(kk, vv[1 % VEC]));
                n.z = __fadd_rn(__fmul_rn(s.z, decay), __fmul_rn(kk, vv[2 % VEC]));
                n.w = __fadd_rn(__fmul_rn(s.w, decay), __fmul_rn(kk, vv[3 % VEC]));
                *reinterpret_cast<float4*>(dst + (size_t)kd * p.Dv + col0) = n;
                o[0] = fmaf(qq, n.x, o[0]);
                o[1 % VEC] = fmaf(qq, n.y, o[1 % VEC]);
                o[2 % VEC] = fmaf(qq, n.z, o[2 % VEC]);
                o[3 % VEC] = fmaf(qq, n.w, o[3 % VEC]);
            }
        }
    } else {
        if (col0 < p.Dv) {
#pragma unroll 4
            for (int kd = rg; kd < p.Dk; kd += RG) {
                const float s = src[(size_t)kd * p.Dv + col0];
                const float n = __fadd_rn(__fmul_rn(s, decay), __fmul_rn(s_k[kd], vv[0]));
                dst[(size_t)kd * p.Dv + col0] = n;
                o[0] = fmaf(s_q[kd], n, o[0]);
            }
        }
    }

#pragma unroll
    for (int j = 0; j < VEC; ++j) s_red[rg][ct * VEC + j] = o[j];
    __syncthreads();
    if (threadIdx.x < kLinCols) {
        const int col = slice * kLinCols + threadIdx.x;
        if (col < p.Dv) {
            float sum = 0.0f;
#pragma unroll 8
            for (int r = 0; r < RG; ++r) sum += s_red[r][threadIdx.x];
            static_cast<T*>(p.out)[((size_t)b * p.Hv + h) * p.Dv + col] = from_float<T>(sum);
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Several consecutive steps in one launch, the state resident on chip.
//
// Same partition (a CTA owns 32 value columns of one (batch, head) state matrix) and the same
// arithmetic in the same order as the single-step kernel, so the outputs and the final state are
// bit-identical to calling it once per step.  The difference is where the state lives: every thread
// keeps its rows x 4 columns of the fp32 state in registers for the whole call; HBM sees the
// state once on the way in and once on the way out, and per step only q, k, v and the output move.
// The next step's q, k, v are fetched while the current step is computed.
// ---------------------------------------------------------------------------------------------
constexpr int kLinStepRows = 8;  // state rows per thread: key_dim <= 8 * 32

struct LinStepsParams {
    const void* q;      // [steps][B][Hk][Dk]
    const void* k;
    const void* v;      // [steps][B][Hv][Dv]
    const float* state;
    void* out;          // [steps][B][Hv][Dv]
    float* new_state;
    const float* decay_ps;  // [steps][B][Hv] or null
    const float* beta_ps;   // [steps][B][Hv] or null
    int steps, B, Hk, Hv, Dk, Dv;
    float decay;
};

template <typename T>
__global__ void __launch_bounds__(kLinThreads) linear_attention_steps_kernel(const LinStepsParams p) {
    constexpr int VEC = 4;
    constexpr int CT = kLinCols / VEC;     // 8 threads across the column slice
    constexpr int RG = kLinThreads / CT;   // 32 row groups
    extern __shared__ float s_dyn[];       // q[Dk], k[Dk]
    __shared__ float s_red[RG][kLinCols + 1];
    __shared__ float s_v[kLinCols];

    const int slices = (p.Dv + kLinCols - 1) / kLinCols;
    const int slice = blockIdx.x % slices;
    const int bh = blockIdx.x / slices;
    const int h = bh % p.Hv;
    const int b = bh / p.Hv;
    const int hk = h / (p.Hv / p.Hk);
    const int tid = threadIdx.x;
    const int ct = tid % CT, rg = tid / CT;
    const int col0 = slice * kLinCols + ct * VEC;
    const bool live = col0 < p.Dv;  // Dv % 4 == 0 on this path

    float* s_q = s_dyn;
    float* s_k = s_dyn + p.Dk;
    const size_t qk_step = (size_t)p.B * p.Hk * p.Dk, v_step = (size_t)p.B * p.Hv * p.Dv, g_step = (size_t)p.B * p.Hv;
    const T* q = static_cast<const T*>(p.q) + ((size_t)b * p.Hk + hk) * p.Dk;
    const T* k = static_cast<const T*>(p.k) + ((size_t)b * p.Hk + hk) * p.Dk;
    const T* v = static_cast<const T*>(p.v) + ((size_t)b * p.Hv + h) * p.Dv + slice * kLinCols;
    T* out = static_cast<T*>(p.out) + ((size_t)b * p.Hv + h) * p.Dv + slice * kLinCols;
    const size_t gidx = (size_t)b * p.Hv + h;

    // the state slice of this thread: rows rg, rg + 32, ... x 4 columns
    const size_t base = ((size_t)b * p.Hv + h) * p.Dk * p.Dv;
    float4 st[kLinStepRows];
#pragma unroll
    for (int r = 0; r < kLinStepRows; ++r) {
        const int kd = rg + r * RG;
        st[r] = (live && kd < p.Dk) ? *reinterpret_cast<const float4*>(p.state + base + (size_t)kd * p.Dv + col0)
                                    : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    // software pipeline: thread i carries element i (and i + 256) of the next step's q and k, and
    // the first 32 threads the next step's v slice
    auto fetch = [&](int step, float (&nq)[2], float (&nk)[2], float& nv) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = tid + j * kLinThreads;
            nq[j] = (i < p.Dk) ? to_float<T>(q[(size_t)step * qk_step + i]) : 0.0f;
            nk[j] = (i < p.Dk) ? to_float<T>(k[(size_t)step * qk_step + i]) : 0.0f;
        }
        nv = (tid < kLinCols && slice * kLinCols + tid < p.Dv) ? to_float<T>(v[(size_t)step * v_step + tid]) : 0.0f;
    };
    float nq[2], nk[2], nv;
    fetch(0, nq, nk, nv);

    for (int step = 0; step < p.steps; ++step) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int i = tid + j * kLinThreads;
            if (i < p.Dk) { s_q[i] = nq[j]; s_k[i] = nk[j]; }
        }
        if (tid < kLinCols) s_v[tid] = nv;
        const float decay = p.decay_ps ? p.decay_ps[(size_t)step * g_step + gidx] : p.decay;
        const float beta = p.beta_ps ? p.beta_ps[(size_t)step * g_step + gidx] : 1.0f;
        __syncthreads();
        if (step + 1 < p.steps) fetch(step + 1, nq, nk, nv);

        float vv[VEC], o[VEC];
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            const float raw = s_v[ct * VEC + j];
            vv[j] = p.beta_ps ? __fmul_rn(raw, beta) : raw;
            o[j] = 0.0f;
        }
        if (live) {
#pragma unroll
            for (int r = 0; r < kLinStepRows; ++r) {
                const int kd = rg + r * RG;
                if (kd < p.Dk) {
                    const float kk = s_k[kd], qq = s_q[kd];
                    float4 n;
                    n.x = __fadd_rn(__fmul_rn(st[r].x, decay), __fmul_rn(kk, vv[0]));
                    n.y = __fadd_rn(__fmul_rn(st[r].y, decay), __fmul_rn(kk, vv[1]));
                    n.z = __fadd_rn(__fmul_rn(st[r].z, decay), __fmul_rn(kk, vv[2]));
                    n.w = __fadd_rn(__fmul_rn(st[r].w, decay), __fmul_rn(kk, vv[3]));
                    st[r] = n;
                    o[0] = fmaf(qq, n.x, o[0]);
                    o[1] = fmaf(qq, n.y, o[1]);
                    o[2] = fmaf(qq, n.z, o[2]);
                    o[3] = fmaf(qq, n.w, o[3]);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < VEC; ++j) s_red[rg][ct * VEC + j] = o[j];
        __syncthreads();
        if (tid < kLinCols && slice * kLinCols + tid < p.Dv) {
            float sum = 0.0f;
#pragma unroll 8
            for (int r = 0; r < RG; ++r) sum += s_red[r][tid];
            out[(size_t)step * v_step + tid] = from_float<T>(sum);
        }
        // the next iteration's writes to s_q / s_k / s_v happen after everyone has passed the barrier
        // above; its writes to s_red come after its own first barrier, i.e. after the sums were read
    }

#pragma unroll
    for (int r = 0; r < kLinStepRows; ++r) {
        const int kd = rg + r * RG;
        if (live && kd < p.Dk) *reinterpret_cast<float4*>(p.new_state + base + (size_t)kd * p.Dv + col0) = st[r];
    }
}

template <typename T>
int launch_linear(const LinParams& p, cudaStream_t stream) {
    const int slices = (p.Dv + kLinCols - 1) / kLinCols;
    const long long ctas = (long long)p.B * p.Hv * slices;
    if (ctas > 0x7fffffffLL) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_attention_decode: too many (batch, head) pairs");
    const size_t smem = (size_t)2 * p.Dk * sizeof(float);
    if (smem > 40 * 1024) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_attention_decode: key_dim %d is too large", p.Dk);
    const bool vec = (p.Dv % 4 == 0) && ((reinterpret_cast<uintptr_t>(p.state) & 15u) == 0) &&
                     ((reinterpret_cast<uintptr_t>(p.new_state) & 15u) == 0);
    if (vec) linear_attention_kernel<T, 4><<<(unsigned)ctas, kLinThreads, smem, stream>>>(p);
    else linear_attention_kernel<T, 1><<<(unsigned)ctas, kLinThreads, smem, stream>>>(p);
    MK36_CUDA_OK(cudaGetLastError());
    return MK36_OK;
}

}  // namespace mk36

using namespace mk36;

extern "C" int mk36_linear_attention_decode(const mk36_linear_attention_args* a, void* stream) {
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode: args is NULL");
    if (!a->q || !a->k || !a->v || !a->state || !a->out || !a->new_state)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode: NULL tensor pointer");
    if (a->batch <= 0 || a->key_heads <= 0 || a->value_heads <= 0 || a->key_dim <= 0 || a->value_dim <= 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode: sizes must be positive");
    if (a->value_heads % a->key_heads != 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode: value_heads must be a multiple of key_heads");
    if (!current_device_info()) return MK36_ERR_LAUNCH;
    LinParams p;
    p.q = a->q;
    p.k = a->k;
    p.v = a->v;
    p.state = a->state;
    p.out = a->out;
    p.new_state = a->new_state;
    p.decay_ph = a->decay_per_head;
    p.beta_ph = a->beta_per_head;
    p.B = a->batch;
    p.Hk = a->key_heads;
    p.Hv = a->value_heads;
    p.Dk = a->key_dim;
    p.Dv = a->value_dim;
    p.decay = a->decay;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (a->dtype) {
        case MK36_BF16: return launch_linear<__nv_bfloat16>(p, s);
        case MK36_F16: return launch_linear<__half>(p, s);
        case MK36_F32: return launch_linear<float>(p, s);
        default: MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_attention_decode: unsupported dtype %d", a->dtype);
    }
}

// Several steps in one call; see the kernel above.  Shapes outside its fast path (value_dim not a
// multiple of 4, key_dim above 256, unaligned state) run the single-step kernel once per step on the
// same stream, with the same results.
extern "C" int mk36_linear_attention_decode_steps(const mk36_linear_attention_steps_args* a, void* stream) {
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode_steps: args is NULL");
    if (!a->q || !a->k || !a->v || !a->state || !a->out || !a->new_state)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode_steps: NULL tensor pointer");
    if (a->steps <= 0 || a->batch <= 0 || a->key_heads <= 0 || a->value_heads <= 0 || a->key_dim <= 0 || a->value_dim <= 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode_steps: sizes must be positive");
    if (a->value_heads % a->key_heads != 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "linear_attention_decode_steps: value_heads must be a multiple of key_heads");
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16 && a->dtype != MK36_F32)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_attention_decode_steps: unsupported dtype %d", a->dtype);
    if (!current_device_info()) return MK36_ERR_LAUNCH;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const bool fast = (a->value_dim % 4 == 0) && a->key_dim <= kLinStepRows * 32 && a->key_dim <= 2 * kLinThreads &&
                      ((reinterpret_cast<uintptr_t>(a->state) & 15u) == 0) && ((reinterpret_cast<uintptr_t>(a->new_state) & 15u) == 0);
    const size_t es = a->dtype == MK36_F32 ? 4 : 2;
    if (!fast) {
        const size_t qk = (size_t)a->batch * a->key_heads * a->key_dim * es, vb = (size_t)a->batch * a->value_heads * a->value_dim * es;
        const size_t gs = (size_t)a->batch * a->value_heads;
        for (int t = 0; t < a->steps; ++t) {
            mk36_linear_attention_args one{};
            one.q = static_cast<const unsigned char*>(a->q) + t * qk;
            one.k = static_cast<const unsigned char*>(a->k) + t * qk;
            one.v = static_cast<const unsigned char*>(a->v) + t * vb;
            one.state = (t == 0) ? a->state : a->new_state;  // in place from the second step on
            one.out = static_cast<unsigned char*>(a->out) + t * vb;
            one.new_state = a->new_state;
            one.decay_per_head = a->decay_per_step ? a->decay_per_step + t * gs : nullptr;
            one.beta_per_head = a->beta_per_step ? a->beta_per_step + t * gs : nullptr;
            one.dtype = a->dtype;
            one.batch = a->batch;
            one.key_heads = a->key_heads;
            one.value_heads = a->value_heads;
            one.key_dim = a->key_dim;
            one.value_dim = a->value_dim;
            one.decay = a->decay;
            const int rc = mk36_linear_attention_decode(&one, stream);
            if (rc != MK36_OK) return rc;
        }
        return MK36_OK;
    }
    LinStepsParams p;
    p.q = a->q; p.k = a->k; p.v = a->v;
    p.state = a->state; p.out = a->out; p.new_state = a->new_state;
    p.decay_ps = a->decay_per_step; p.beta_ps = a->beta_per_step;
    p.steps = a->steps; p.B = a->batch; p.Hk = a->key_heads; p.Hv = a->value_heads; p.Dk = a->key_dim; p.Dv = a->value_dim;
    p.decay = a->decay;
    const int slices = (p.Dv + kLinCols - 1) / kLinCols;
    const long long ctas = (long long)p.B * p.Hv * slices;
    if (ctas > 0x7fffffffLL) MK36_FAIL(MK36_ERR_UNSUPPORTED, "linear_attention_decode_steps: too many (batch, head) pairs");
    const size_t smem = (size_t)2 * p.Dk * sizeof(float);
    switch (a->dtype) {
        case MK36_BF16: linear_attention_steps_kernel<__nv_bfloat16><<<(unsigned)ctas, kLinThreads, smem, s>>>(p); break;
        case MK36_F16: linear_attention_steps_kernel<__half><<<(unsigned)ctas, kLinThreads, smem, s>>>(p); break;
        default: linear_attention_steps_kernel<float><<<(unsigned)ctas, kLinThreads, smem, s>>>(p); break;
    }
    MK36_CUDA_OK(cudaGetLastError());
    return MK36_OK;
}
