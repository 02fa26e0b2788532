// Dense SwiGLU FFN decode on warp-level tensor-core instructions, weights streamed from HBM straight
// into MMA fragments (2-byte dtypes, up to 8 tokens per launch).
//
// out = x + Wd (silu(Wg n) * (Wu n)),  n = RMSNorm(x)       (mega_kernel_qwen36/reference.py:65-88)
//
// With up to eight tokens the three weight matrices dominate everything (535 MB at the 27B shape), and
// the tokens are the N = 8 columns of mma.sync.m16n8k16, so one pass over the weights serves the
// whole batch.  The weights never touch shared memory: lane (g, t) of a warp loads 16 bytes of
// rows g and g + 8 of its tile directly from global memory in the order the instruction wants
// (contraction index permuted identically on both operands, see mk36_mma.cuh), several slices
// ahead of the MMAs, and each warp walks its rows sequentially along the contraction, which keeps
// the DRAM pages open.
//
//   phase 0  every CTA normalises the tokens into shared memory (rounded to the storage dtype, as
//            the reference does), columns beyond the batch are zero
//   phase A  tile = 8 gate rows (fragment rows 0-7) + the 8 matching up rows (fragment rows 8-15),
//            one warp per tile over the whole hidden length; gate and up of a channel end up in
//            the same thread, which writes silu(g) * u as fp32 to the workspace
//   grid barrier
//   phase C  the CTA owns output rows [h0, h1) (up to three 16-row tiles); each warp takes a
//            contiguous range of the intermediate length for all tiles, reads the fp32
//            activations of its range from L2, splits them into a high and a low half in the
//            storage dtype (two MMAs, nothing lost) and accumulates; the warps' partial tiles meet in
//            shared memory; residual, rounding, store (or the cross-GPU exchange)
#include "mk36_comm.cuh"
#include "mk36_mma.cuh"

namespace mk36 {

constexpr int kDenseWarps = 16;
constexpr int kDenseThreads = kDenseWarps * 32;
constexpr int kDenseMaxTokens = 8;
constexpr int kDenseMaxTiles = 3;   // 16-row output tiles per CTA
constexpr int kDenseAhead = 8;      // 32-wide slices of phase A in flight per warp

struct DenseMmaParams {
    const void* x;
    const void* norm_w;
    const void* gate;
    const void* up;
    const void* down;
    void* out;
    float* partial_out;
    Control* ctl;
    float* act;   // [8][I] fp32 scratch
    int ntok, H, I, add_residual;
    float eps;
    CommParams comm;
};

__device__ __forceinline__ uint4 ldg_stream(const void* p) { return ld_stream_u4(p); }

// fp32 values of 8 consecutive channels -> high and low halves in T, packed like a weight load
template <typename T>
__device__ __forceinline__ void split_hi_lo(const float4& a, const float4& b, uint4& hi, uint4& lo) {
    const float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    T h[8], l[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        h[i] = from_float<T>(v[i]);
        l[i] = from_float<T>(v[i] - to_float<T>(h[i]));
    }
    hi = *reinterpret_cast<const uint4*>(h);
    lo = *reinterpret_cast<const uint4*>(l);
}

template <typename T>
__global__ void __launch_bounds__(kDenseThreads, 1) dense_ffn_mma_kernel(const DenseMmaParams p) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ unsigned s_step;
    T* xs = reinterpret_cast<T*>(smem);               // [8][H], tokens beyond ntok are zero
    float* red = reinterpret_cast<float*>(smem);      // phase C: [warps][tiles][128] partial tiles (reuses xs)

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t = lane & 3;
    const int cta = blockIdx.x, ncta = gridDim.x;
    const bool exchange = p.comm.world > 1;
    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);
    if (tid == 0) s_step = exchange ? comm_read_step(p.comm) : 0u;

    const T* x = static_cast<const T*>(p.x);
    const T* nw = static_cast<const T*>(p.norm_w);
    const size_t H = (size_t)p.H, I = (size_t)p.I;

    // ---- phase 0: RMSNorm; the 16 warps are shared out over the tokens (16, 8, 4 or 2 warps per token) ----
    {
        __shared__ float s_part[kDenseWarps];
        int tp2 = 1;
        while (tp2 < p.ntok) tp2 <<= 1;
        const int wpt = kDenseWarps / tp2;          // warps per token
        const int b = warp / wpt, part = warp - b * wpt;
        const int nchunk = p.H >> 3, stride = wpt * 32;
        const bool live = b < p.ntok;
        const T* xr = x + (size_t)(live ? b : 0) * H;
        float ss = 0.0f;
        if (live) {
            for (int c = part * 32 + lane; c < nchunk; c += stride) {
                Chunk8<T> v;
                v.raw = *reinterpret_cast<const uint4*>(xr + 8 * c);
                float f[8];
                unpack8(v, f);
#pragma unroll
                for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
            }
        }
        ss = warp_sum(ss);
        if (lane == 0) s_part[warp] = ss;
        // columns beyond the batch are zero
        for (int idx = tid; idx < (kDenseMaxTokens - p.ntok) * nchunk; idx += kDenseThreads)
            *reinterpret_cast<uint4*>(xs + (size_t)p.ntok * H + 8 * (size_t)idx) = make_uint4(0, 0, 0, 0);
        __syncthreads();
        if (live) {
            float tot = 0.0f;
            for (int w = 0; w < wpt; ++w) tot += s_part[b * wpt + w];
            const float rstd = 1.0f / sqrtf(tot / (float)p.H + p.eps);
            T* dst = xs + (size_t)b * H;
            for (int c = part * 32 + lane; c < nchunk; c += stride) {
                Chunk8<T> v, w;
                v.raw = *reinterpret_cast<const uint4*>(xr + 8 * c);
                w.raw = *reinterpret_cast<const uint4*>(nw + 8 * c);
                float f[8], wf[8];
                unpack8(v, f);
                unpack8(w, wf);
                T o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(f[i], rstd), wf[i]));
                *reinterpret_cast<uint4*>(dst + 8 * c) = *reinterpret_cast<const uint4*>(o);
            }
        }
    }
    __syncthreads();
    if (tracer) trace_stamp(p.ctl, 1);

    // ---- phase A: gate/up tiles ----
    // The CTA owns a contiguous range of tiles.  When it has fewer tiles than warps (a tensor-parallel
    // shard), ks = 2, 4, 8 or 16 warps share a tile and split the hidden length, so that all warps keep
    // streaming; their partial sums meet in shared memory before SiLU.
    {
        __shared__ float4 s_parta[kDenseThreads];
        const T* gw = static_cast<const T*>(p.gate);
        const T* uw = static_cast<const T*>(p.up);
        const int ntiles = p.I >> 3;
        const int nsl = p.H >> 5;  // 32-wide slices of the contraction
        const int t_lo = (int)(((long long)ntiles * cta) / ncta), t_hi = (int)(((long long)ntiles * (cta + 1)) / ncta);
        const int nt = t_hi - t_lo;
        int ks = 1;
        while (ks < kDenseWarps && nt * (ks * 2) <= kDenseWarps) ks <<= 1;
        const int per_round = kDenseWarps / ks;
        const int kpart = warp & (ks - 1), tslot = warp / ks;
        const int sa = (int)(((long long)nsl * kpart) / ks), sb = (int)(((long long)nsl * (kpart + 1)) / ks);
        const T* bcol = xs + (size_t)g * H + 8 * t;
        for (int r0 = 0; r0 < nt; r0 += per_round) {  // the same trip count for every warp of the CTA
            const bool live = r0 + tslot < nt;
            const int tile = t_lo + (live ? r0 + tslot : 0);
            const T* ga = gw + ((size_t)tile * 8 + g) * H + 8 * t;
            const T* ua = uw + ((size_t)tile * 8 + g) * H + 8 * t;
            float d0[4] = {0.f, 0.f, 0.f, 0.f}, d1[4] = {0.f, 0.f, 0.f, 0.f};
            if (live) {
                uint4 qa[kDenseAhead], qb[kDenseAhead];
#pragma unroll
                for (int j = 0; j < kDenseAhead; ++j) {
                    if (sa + j < sb) {
                        qa[j] = ldg_stream(ga + 32 * (sa + j));
                        qb[j] = ldg_stream(ua + 32 * (sa + j));
                    }
                }
                for (int s0 = sa; s0 < sb; s0 += kDenseAhead) {
#pragma unroll
                    for (int j = 0; j < kDenseAhead; ++j) {
                        const int s = s0 + j;
                        if (s < sb) {
                            const uint4 a = qa[j], b = qb[j];
                            const int nx = s + kDenseAhead;
                            if (nx < sb) {  // refill this slot before using its old contents
                                qa[j] = ldg_stream(ga + 32 * nx);
                                qb[j] = ldg_stream(ua + 32 * nx);
                            }
                            const uint4 xv = *reinterpret_cast<const uint4*>(bcol + 32 * s);
                            mma_slice32<T>(d0, d1, a, b, xv);
                        }
                    }
                }
            }
            // rows g (gate) and g + 8 (up) of channel 8 * tile + g, tokens 2t and 2t + 1
            float g0 = d0[0] + d1[0], g1 = d0[1] + d1[1], u0 = d0[2] + d1[2], u1 = d0[3] + d1[3];
            if (ks > 1) {
                s_parta[tid] = make_float4(g0, g1, u0, u1);
                __syncthreads();
                if (kpart == 0) {
                    for (int q = 1; q < ks; ++q) {
                        const float4 o = s_parta[tid + 32 * q];
                        g0 += o.x; g1 += o.y; u0 += o.z; u1 += o.w;
                    }
                }
                __syncthreads();  // the partials have been read before the next round overwrites them
            }
            if (live && kpart == 0) {
                const int ch = tile * 8 + g;
                if (2 * t < p.ntok) p.act[(size_t)(2 * t) * I + ch] = silu(g0) * u0;
                if (2 * t + 1 < p.ntok) p.act[(size_t)(2 * t + 1) * I + ch] = silu(g1) * u1;
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 2);

    // ---- grid barrier: all activations are in the workspace ----
    if (!grid_barrier(p.ctl, ncta, 0u, kStatusDenseBarrier, &s_flag)) return;
    if (tid == 0) barrier_finish(p.ctl, ncta);
    if (tracer) trace_stamp(p.ctl, 3);

    // ---- phase C: down rows of this CTA ----
    const int h0 = (int)(((long long)p.H * cta) / ncta);
    const int h1 = (int)(((long long)p.H * (cta + 1)) / ncta);
    const int hr = h1 - h0;
    const int ntile = (hr + 15) >> 4;
    float acc[kDenseMaxTiles][2][4];
#pragma unroll
    for (int i = 0; i < kDenseMaxTiles; ++i)
#pragma unroll
        for (int j = 0; j < 2; ++j) { acc[i][j][0] = 0.f; acc[i][j][1] = 0.f; acc[i][j][2] = 0.f; acc[i][j][3] = 0.f; }
    {
        const T* dw = static_cast<const T*>(p.down);
        const int nsl = p.I >> 5;
        const int sl0 = (int)(((long long)nsl * warp) / kDenseWarps), sl1 = (int)(((long long)nsl * (warp + 1)) / kDenseWarps);
        const uint4 zero = make_uint4(0, 0, 0, 0);
        const T* rlo[kDenseMaxTiles];
        const T* rhi[kDenseMaxTiles];
        bool vlo[kDenseMaxTiles], vhi[kDenseMaxTiles];
#pragma unroll
        for (int i = 0; i < kDenseMaxTiles; ++i) {
            const int r = 16 * i + g;
            vlo[i] = i < ntile && r < hr;
            vhi[i] = i < ntile && r + 8 < hr;
            rlo[i] = dw + (size_t)(h0 + (vlo[i] ? r : 0)) * I + 8 * t;
            rhi[i] = dw + (size_t)(h0 + (vhi[i] ? r + 8 : 0)) * I + 8 * t;
        }
        const float* arow = p.act + (size_t)g * I + 8 * t;  // token g's activations (zero weights beyond ntok do not matter:
        const bool col = g < p.ntok;                        //  columns beyond the batch are never stored)
        // two slices in flight per warp (explicit double buffer; slot j is refilled right after its use)
        uint4 wa[2][kDenseMaxTiles], wb[2][kDenseMaxTiles];
        float4 fa[2], fb[2];
        auto fetch = [&](int slot, int s) {
#pragma unroll
            for (int i = 0; i < kDenseMaxTiles; ++i) {
                wa[slot][i] = vlo[i] ? ldg_stream(rlo[i] + 32 * s) : zero;
                wb[slot][i] = vhi[i] ? ldg_stream(rhi[i] + 32 * s) : zero;
            }
            fa[slot] = make_float4(0.f, 0.f, 0.f, 0.f);
            fb[slot] = fa[slot];
            if (col) {
                fa[slot] = __ldcg(reinterpret_cast<const float4*>(arow + 32 * s));
                fb[slot] = __ldcg(reinterpret_cast<const float4*>(arow + 32 * s + 4));
            }
        };
#pragma unroll
        for (int j = 0; j < 2; ++j)
            if (sl0 + j < sl1) fetch(j, sl0 + j);
        for (int s0 = sl0; s0 < sl1; s0 += 2) {
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int s = s0 + j;
                if (s < sl1) {
                    uint4 hi, lo;
                    split_hi_lo<T>(fa[j], fb[j], hi, lo);
#pragma unroll
                    for (int i = 0; i < kDenseMaxTiles; ++i) {
                        if (i < ntile) {
                            mma_slice32<T>(acc[i][0], acc[i][1], wa[j][i], wb[j][i], hi);
                            mma_slice32<T>(acc[i][0], acc[i][1], wa[j][i], wb[j][i], lo);
                        }
                    }
                    if (s + 2 < sl1) fetch(j, s + 2);
                }
            }
        }
    }
    if (tracer) trace_stamp(p.ctl, 4);

    // ---- the warps' partial tiles meet in shared memory ----
    __syncthreads();  // the token vectors in shared memory are no longer needed
#pragma unroll
    for (int i = 0; i < kDenseMaxTiles; ++i) {
        if (i < ntile) {
            float* mine = red + ((size_t)warp * kDenseMaxTiles + i) * 128;
            *reinterpret_cast<float2*>(mine + g * 8 + 2 * t) = make_float2(acc[i][0][0] + acc[i][1][0], acc[i][0][1] + acc[i][1][1]);
            *reinterpret_cast<float2*>(mine + (g + 8) * 8 + 2 * t) = make_float2(acc[i][0][2] + acc[i][1][2], acc[i][0][3] + acc[i][1][3]);
        }
    }
    __syncthreads();
    T* out = static_cast<T*>(p.out);
    const unsigned step = s_step;
    for (int idx = tid; idx < hr * 8; idx += kDenseThreads) {
        const int r = idx >> 3, c = idx & 7;
        if (c >= p.ntok) continue;
        const int tile = r >> 4, rr = r & 15;
        float v = 0.0f;
#pragma unroll
        for (int w = 0; w < kDenseWarps; ++w) v += red[((size_t)w * kDenseMaxTiles + tile) * 128 + rr * 8 + c];
        const size_t o = (size_t)c * H + h0 + r;
        if (exchange) {
            comm_put(p.comm, step, o, v);
        } else if (p.partial_out) {
            p.partial_out[o] = v;
        } else {
            if (p.add_residual) v += to_float<T>(x[o]);
            out[o] = from_float<T>(v);
        }
    }
    if (exchange) {
        for (int idx = tid; idx < hr * 8; idx += kDenseThreads) {
            const int r = idx >> 3, c = idx & 7;
            if (c >= p.ntok) continue;
            const size_t o = (size_t)c * H + h0 + r;
            float v;
            if (!comm_get_sum(p.comm, p.ctl, step, o, &v)) continue;
            if (p.add_residual) v += to_float<T>(x[o]);
            out[o] = from_float<T>(v);
        }
        if (cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);  // every CTA read it before the grid barrier
    }
    if (tracer) trace_stamp(p.ctl, 5);
}

// Launches the tensor-core variant when the shapes suit it and sets *handled; otherwise leaves
// *handled false (no error) and the caller uses the general kernel.
int dense_ffn_mma_launch(const mk36_dense_ffn_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                         bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    const int H = a->hidden, I = a->intermediate;
    if (H % 32 != 0 || I % 32 != 0) return MK36_OK;
    const void* ptrs[] = {a->x, a->norm_weight, a->gate_weight, a->up_weight, a->down_weight};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const int ncta = dev->sm_count;
    const int hr_max = (H + ncta - 1) / ncta;
    if (hr_max > 16 * kDenseMaxTiles) return MK36_OK;
    const size_t xs_bytes = (size_t)kDenseMaxTokens * H * 2;
    const size_t red_bytes = (size_t)kDenseWarps * kDenseMaxTiles * 128 * 4;
    const size_t smem = xs_bytes > red_bytes ? xs_bytes : red_bytes;
    if (smem + 1024 > (size_t)dev->max_smem_optin) return MK36_OK;

    DenseMmaParams p;
    int rc = comm_params_from(comm, H, &p.comm, "dense_ffn_decode");
    if (rc != MK36_OK) return rc;
    if (p.comm.world > 1 && (!a->out || a->partial_out))
        MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: the multi-GPU entry point writes `out` and takes no partial_out");
    const size_t scratch = align_up((size_t)kDenseMaxTokens * I * 4, 256);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "dense_ffn_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + scratch)
        MK36_FAIL(MK36_ERR_WORKSPACE, "dense_ffn_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, kControlBytes + scratch);

    p.norm_w = a->norm_weight;
    p.gate = a->gate_weight;
    p.up = a->up_weight;
    p.down = a->down_weight;
    p.ctl = static_cast<Control*>(workspace);
    p.act = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kControlBytes);
    p.H = H;
    p.I = I;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    const void* kernel = (a->dtype == MK36_BF16) ? (const void*)dense_ffn_mma_kernel<__nv_bfloat16> : (const void*)dense_ffn_mma_kernel<__half>;
    rc = ensure_dynamic_smem(kernel, smem);
    if (rc != MK36_OK) return rc;
    for (int b0 = 0; b0 < a->batch; b0 += kDenseMaxTokens) {
        p.ntok = (a->batch - b0 < kDenseMaxTokens) ? (a->batch - b0) : kDenseMaxTokens;
        p.x = static_cast<const unsigned char*>(a->x) + (size_t)b0 * H * 2;
        p.out = a->out ? static_cast<unsigned char*>(a->out) + (size_t)b0 * H * 2 : nullptr;
        p.partial_out = a->partial_out ? a->partial_out + (size_t)b0 * H : nullptr;
        void* params[] = {&p};
        rc = launch_cooperative(kernel, dim3(ncta), dim3(kDenseThreads), smem, stream, params, "dense_ffn_decode(mma)");
        if (rc != MK36_OK) return rc;
    }
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
