// Dense SwiGLU FFN decode for ONE token on sm_100a (2-byte dtypes, aligned shapes): RMSNorm ->
// silu(x Wg^T) * (x Wu^T) -> Wd -> residual, arithmetic of mega_kernel_qwen36/reference.py:65-88.
// Replaces the three library GEMVs of the reference's GPU path (mega_kernel_qwen36/ops.py:202-218).
//
// With one token the op is a pure weight stream (535 MB at the 27B shape) and its speed is the
// number of bytes a CTA keeps in flight.  Loads staged in registers cap that at what the register
// file holds (about 128 KB per SM, ~4.5 TB/s); here the weights never pass through registers on
// their way in: one producer lane feeds a shared-memory ring with 1-D bulk copies (cp.async.bulk
// completing on mbarriers, each copy into the issuing CTA only), 160 - 200 KB per SM in flight.
//
//   phase A   chunk = two (gate, up) row pairs = two contiguous gate rows + the two matching up rows
//             (4 x hidden elements); a warp takes a pair, so silu(g) * u is formed without a trip
//             through memory; results -> global scratch.  The chunks are dealt to the CTAs: the
//             first rounds statically, the rest through a work counter, so that a CTA whose memory
//             is served faster takes more and all reach the grid barrier together
//   grid barrier (the only one; the first down rows are requested before it completes)
//   phase C   chunk = one down row (intermediate elements); three warps share a row, their partial
//             sums meet in shared memory; residual, rounding, store (or the cross-GPU exchange)
//
// Chunk c lives in stage c % depth of its phase's ring.  Every consumer warp waits for every chunk
// and releases it, so that all warps see every barrier phase exactly once, in order (a warp that
// skipped phases could mistake an older phase for the one it waits for).  In phase A the producer
// writes what a stage holds (first channel, pairs; no pairs = the stream has ended) next to it
// before it arms the stage, because with dealt chunks the consumers cannot compute it.  The two rings share the
// same shared memory: phase C's activations and ring lie over phase A's token and ring, and the
// producer requests the first down row only after phase A's last chunk has been released.
//
// Plain FMAs with warp-shuffle reductions: with one token column a tensor-core tile would be all
// padding.  Batches of two or more tokens take the tensor-core kernel in dense_ffn_mma.cu.
#include "mk36_comm.cuh"
#include "mk36_ring.cuh"

namespace mk36 {

constexpr int kDsConsumerWarps = 12;  // + 1 producer: 13 warps are allocated as 16, i.e. 128 registers per thread
constexpr int kDsConsumerThreads = kDsConsumerWarps * 32;
constexpr int kDsThreads = kDsConsumerThreads + 32;
constexpr int kDsPairsPerChunk = 2;
constexpr int kDsWarpsPerRow = 3;     // phase C: warps that share a down row
constexpr int kDsRowGroups = kDsConsumerWarps / kDsWarpsPerRow;
constexpr int kDsMaxStages = 8;

struct DenseStreamParams {
    const void* x;
    const void* norm_w;
    const void* gate;
    const void* up;
    const void* down;
    void* out;
    float* partial_out;
    Control* ctl;
    float* act;  // [I] silu(gate) * up, fp32, global scratch
    int H, I, add_residual;
    float eps;
    int ra, rc;                  // ring depths of the two phases
    int stage_a_bytes, stage_c_bytes;
    FastDiv fd_ncta;
    int deal_static;  // 1: no work counter
    int off_bars, off_red, off_desc, off_base, off_ring_a, off_ring_c;
    CommParams comm;
};

template <typename T>
__device__ __forceinline__ void ds_unpack(const uint4& v, float (&f)[8]) {
    Chunk8<T> c;
    c.raw = v;
    unpack8(c, f);
}

template <typename T>
__global__ void __launch_bounds__(kDsThreads, 1) dense_ffn_stream_kernel(const DenseStreamParams p) {
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ int s_flag;
    __shared__ int s_abort;
    __shared__ unsigned s_step;
    __shared__ float s_red[kDsConsumerWarps];

    const int tid = threadIdx.x;
    const int lane = tid & 31;
    const int warp = tid >> 5;
    const int ncta = gridDim.x;
    const int cta = blockIdx.x;
    const bool is_producer = (warp == kDsConsumerWarps);

    unsigned long long* full_a = reinterpret_cast<unsigned long long*>(smem + p.off_bars);
    unsigned long long* empty_a = full_a + kDsMaxStages;
    unsigned long long* full_c = empty_a + kDsMaxStages;
    unsigned long long* empty_c = full_c + kDsMaxStages;
    float* red = reinterpret_cast<float*>(smem + p.off_red);      // [row groups][warps per row]
    int2* desc = reinterpret_cast<int2*>(smem + p.off_desc);      // phase A, per stage: {first channel, pairs}
    T* xs = reinterpret_cast<T*>(smem + p.off_base);               // phase A: the normalised token as T [H]
    float* acts = reinterpret_cast<float*>(smem + p.off_base);     // phase C: activations, fp32 [I]
    unsigned char* ring_a = smem + p.off_ring_a;
    unsigned char* ring_c = smem + p.off_ring_c;

    const T* x = static_cast<const T*>(p.x);
    const size_t rowH = (size_t)p.H, rowI = (size_t)p.I;
    // ---- static partition: intermediate channels (phase A) and output rows (phase C) of this CTA ----
    const int h0 = fdiv(p.H * cta, p.fd_ncta), h1 = fdiv(p.H * (cta + 1), p.fd_ncta);
    const int n_c = h1 - h0;
    const int chunks_all = (p.I + kDsPairsPerChunk - 1) / kDsPairsPerChunk;

    const bool tracer = (cta == 0 && tid == 0);
    if (tracer) trace_stamp(p.ctl, 0);
    if (tid < 4 * kDsMaxStages) {
        const int which = tid / kDsMaxStages;  // 0 full A, 1 empty A, 2 full C, 3 empty C
        mbar_init(&full_a[tid], (which & 1) ? kDsConsumerWarps : 1);
    }
    if (tid == 0) {
        s_abort = 0;
        s_step = (p.comm.world > 1) ? comm_read_step(p.comm) : 0u;
    }
    if (tid < 32) mbar_init_fence();
    __syncthreads();

    // =====================================================================================
    // Producer warp: one lane issues every copy
    // =====================================================================================
    if (is_producer) {
        if (lane != 0) return;
        // on a workspace whose status word is set nothing may run (and a CTA that leaves must have no copy in flight)
        if (ld_volatile_s32(&p.ctl->status) != 0) {
            *(volatile int*)&s_abort = 1;
            return;
        }
        bool ok = true;
        const size_t row_a = rowH * sizeof(T);
        int stage = 0, use = 0, n_a = 0;
        {
            // the first rounds are dealt statically (no counter traffic while everybody starts), the rest through
            // the counter
            int static_rounds = fdiv(chunks_all, p.fd_ncta);
            if (!p.deal_static) static_rounds = max(static_rounds - 3, 0);
            const int dyn_base = static_rounds * ncta;
            int k = 0;
            int t_next = (k < static_rounds || p.deal_static) ? cta : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
            for (;;) {
                const int t = t_next;
                const bool last = t >= chunks_all;
                if (!last) {
                    ++k;
                    // the next ticket is in flight while this chunk waits for its stage
                    t_next = (k < static_rounds || p.deal_static) ? k * ncta + cta : dyn_base + (int)atomicAdd(&p.ctl->work_ticket, 1u);
                }
                if (use > 0) ok = mbar_wait(&empty_a[stage], (unsigned)(use - 1) & 1u, &s_abort);
                if (!ok) break;
                ++n_a;
                if (last) {
                    // an empty chunk tells the consumers that the stream of this CTA has ended
                    desc[stage] = make_int2(0, 0);
                    mbar_arrive(&full_a[stage]);
                    if (++stage == p.ra) { stage = 0; ++use; }
                    break;
                }
                const int first = t * kDsPairsPerChunk;
                const int count = min(kDsPairsPerChunk, p.I - first);
                unsigned char* dst = ring_a + (size_t)stage * p.stage_a_bytes;
                const unsigned bytes = (unsigned)(count * row_a);
                desc[stage] = make_int2(first, count);
                mbar_arrive_expect_tx(&full_a[stage], 2 * bytes);
                bulk_copy_g2s(dst, static_cast<const T*>(p.gate) + (size_t)first * rowH, bytes, &full_a[stage]);
                bulk_copy_g2s(dst + kDsPairsPerChunk * row_a, static_cast<const T*>(p.up) + (size_t)first * rowH, bytes, &full_a[stage]);
                if (++stage == p.ra) { stage = 0; ++use; }
            }
        }
        // phase C lies over phase A's shared memory: every stage of phase A must have been released for the last time
        for (int s = 0; s < p.ra && ok; ++s) {
            const int uses = (n_a > s) ? (n_a - 1 - s) / p.ra + 1 : 0;  // how often stage s was filled
            if (uses > 0) ok = mbar_wait(&empty_a[s], (unsigned)(uses - 1) & 1u, &s_abort);
        }
        if (cta == 0) trace_stamp(p.ctl, 10);
        const unsigned row_c = (unsigned)(rowI * sizeof(T));
        stage = 0;
        use = 0;
        for (int c = 0; c < n_c && ok; ++c) {
            if (use > 0) ok = mbar_wait(&empty_c[stage], (unsigned)(use - 1) & 1u, &s_abort);
            if (!ok) break;
            mbar_arrive_expect_tx(&full_c[stage], row_c);
            bulk_copy_g2s(ring_c + (size_t)stage * p.stage_c_bytes, static_cast<const T*>(p.down) + (size_t)(h0 + c) * rowI, row_c, &full_c[stage]);
            if (++stage == p.rc) { stage = 0; ++use; }
        }
        if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingProducer);
        // consumers wait on every barrier that was armed, and a wait only runs out long after any copy has landed
        return;
    }

    // =====================================================================================
    // Consumer warps
    // =====================================================================================
    // ---- RMSNorm of the token into shared memory (as T: the reference rounds the normalised input).  x and the
    //      norm weight are requested together and stay in registers between the two passes. ----
    {
        constexpr int kPer = 4;  // 16-byte pieces per thread held in registers: hidden <= 12288
        uint4 xv[kPer], wv[kPer];
        float ss = 0.0f;
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            const int k = (tid + q * kDsConsumerThreads) * 8;
            xv[q] = make_uint4(0, 0, 0, 0);
            wv[q] = xv[q];
            if (k < p.H) {
                xv[q] = *reinterpret_cast<const uint4*>(x + k);
                wv[q] = *reinterpret_cast<const uint4*>(static_cast<const T*>(p.norm_w) + k);
            }
        }
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            float f[8];
            ds_unpack<T>(xv[q], f);
#pragma unroll
            for (int i = 0; i < 8; ++i) ss = fmaf(f[i], f[i], ss);
        }
        ss = warp_sum(ss);
        if (lane == 0) s_red[warp] = ss;
        named_barrier(1, kDsConsumerThreads);
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < kDsConsumerWarps; ++w) tot += s_red[w];
        const float rstd = 1.0f / sqrtf(tot / (float)p.H + p.eps);
#pragma unroll
        for (int q = 0; q < kPer; ++q) {
            const int k = (tid + q * kDsConsumerThreads) * 8;
            if (k < p.H) {
                float f[8], g[8];
                ds_unpack<T>(xv[q], f);
                ds_unpack<T>(wv[q], g);
                T o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = from_float<T>(__fmul_rn(__fmul_rn(f[i], rstd), g[i]));
                *reinterpret_cast<uint4*>(xs + k) = *reinterpret_cast<const uint4*>(o);
            }
        }
        named_barrier(1, kDsConsumerThreads);
    }
    if (tracer) trace_stamp(p.ctl, 1);

    bool ok = true;
    // ---- phase A: chunk c is worked on by the warp pair (2c, 2c + 1) mod 12, one (gate, up) pair per warp ----
    {
        const int nch = p.H >> 3;
        int stage = 0, use = 0, turn = 0;  // turn = (2 c) mod 12
        for (;;) {
            if (ok) ok = mbar_wait(&full_a[stage], (unsigned)use & 1u, &s_abort);
            if (!ok) break;
            const int2 d = desc[stage];
            if (d.y == 0) {  // the producer's end mark: released like a chunk, then the phase is over
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_a[stage]);
                break;
            }
            const int mine = warp - turn;  // 0 or 1: this warp's pair of the chunk
            if (mine == 0 || mine == 1) {
                const int first = d.x;
                if (mine < d.y) {
                    const T* g = reinterpret_cast<const T*>(ring_a + (size_t)stage * p.stage_a_bytes) + (size_t)mine * rowH;
                    const T* u = g + (size_t)kDsPairsPerChunk * rowH;
                    float sg = 0.0f, su = 0.0f, sg2 = 0.0f, su2 = 0.0f;
                    int k = lane;
                    for (; k + 32 < nch; k += 64) {
                        float fg[8], fu[8], fx[8], hg[8], hu[8], hx[8];
                        ds_unpack<T>(lds128(g + 8 * k), fg);
                        ds_unpack<T>(lds128(u + 8 * k), fu);
                        ds_unpack<T>(lds128(xs + 8 * k), fx);
                        ds_unpack<T>(lds128(g + 8 * (k + 32)), hg);
                        ds_unpack<T>(lds128(u + 8 * (k + 32)), hu);
                        ds_unpack<T>(lds128(xs + 8 * (k + 32)), hx);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            sg = fmaf(fg[i], fx[i], sg);
                            su = fmaf(fu[i], fx[i], su);
                            sg2 = fmaf(hg[i], hx[i], sg2);
                            su2 = fmaf(hu[i], hx[i], su2);
                        }
                    }
                    for (; k < nch; k += 32) {
                        float fg[8], fu[8], fx[8];
                        ds_unpack<T>(lds128(g + 8 * k), fg);
                        ds_unpack<T>(lds128(u + 8 * k), fu);
                        ds_unpack<T>(lds128(xs + 8 * k), fx);
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            sg = fmaf(fg[i], fx[i], sg);
                            su = fmaf(fu[i], fx[i], su);
                        }
                    }
                    sg = warp_sum(sg + sg2);
                    su = warp_sum(su + su2);
                    if (lane == 0) p.act[first + mine] = silu(sg) * su;
                }
            }
            // every warp releases every chunk
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty_a[stage]);
            if (++stage == p.ra) { stage = 0; ++use; }
            turn += kDsPairsPerChunk;
            if (turn >= kDsConsumerWarps) turn -= kDsConsumerWarps;
        }
    }
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    if (tracer) trace_stamp(p.ctl, 2);

    // ---- grid barrier: every CTA's activations are in the scratch buffer ----
    named_barrier(1, kDsConsumerThreads);
    if (tid == 0) {
        bool fine = (*(volatile int*)&s_abort == 0);
        if (fine) {
            const unsigned target = barrier_arrive(p.ctl, ncta, 0);
            fine = barrier_wait(p.ctl, target, kStatusDenseBarrier);
            if (fine) barrier_finish(p.ctl, ncta);
        }
        if (!fine) *(volatile int*)&s_abort = 1;
        s_flag = fine ? 1 : 0;
    }
    named_barrier(1, kDsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 3);
    if (!s_flag) return;

    // ---- all activations into shared memory (over the token and phase A's ring, which are dead now) ----
    for (int k = tid * 4; k < p.I; k += kDsConsumerThreads * 16) {
        float4 v[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int kk = k + q * kDsConsumerThreads * 4;
            if (kk < p.I) v[q] = __ldcg(reinterpret_cast<const float4*>(p.act + kk));
        }
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int kk = k + q * kDsConsumerThreads * 4;
            if (kk < p.I) *reinterpret_cast<float4*>(acts + kk) = v[q];
        }
    }
    named_barrier(1, kDsConsumerThreads);
    if (tracer) trace_stamp(p.ctl, 4);

    // ---- phase C: row c is worked on by row group c mod 4 (three warps, a third of the row each) ----
    T* out = static_cast<T*>(p.out);
    const bool exchange = p.comm.world > 1;
    const unsigned step = s_step;
    {
        const int group = warp / kDsWarpsPerRow, wj = warp % kDsWarpsPerRow;
        const int nch = p.I >> 3;
        const int k_begin = (nch * wj) / kDsWarpsPerRow, k_end = (nch * (wj + 1)) / kDsWarpsPerRow;
        int stage = 0, use = 0, turn = 0;  // turn = c mod 4
        for (int c = 0; c < n_c; ++c) {
            if (ok) ok = mbar_wait(&full_c[stage], (unsigned)use & 1u, &s_abort);
            const bool mine = (turn == group);
            float s0 = 0.0f, s1 = 0.0f;
            if (ok && mine) {
                const T* w = reinterpret_cast<const T*>(ring_c + (size_t)stage * p.stage_c_bytes);
                int k = k_begin + lane;
                for (; k + 32 < k_end; k += 64) {
                    float f[8], h[8];
                    ds_unpack<T>(lds128(w + 8 * k), f);
                    ds_unpack<T>(lds128(w + 8 * (k + 32)), h);
                    const float4 a0 = *reinterpret_cast<const float4*>(acts + 8 * k);
                    const float4 a1 = *reinterpret_cast<const float4*>(acts + 8 * k + 4);
                    const float4 b0 = *reinterpret_cast<const float4*>(acts + 8 * (k + 32));
                    const float4 b1 = *reinterpret_cast<const float4*>(acts + 8 * (k + 32) + 4);
                    s0 = fmaf(f[0], a0.x, s0); s1 = fmaf(h[0], b0.x, s1);
                    s0 = fmaf(f[1], a0.y, s0); s1 = fmaf(h[1], b0.y, s1);
                    s0 = fmaf(f[2], a0.z, s0); s1 = fmaf(h[2], b0.z, s1);
                    s0 = fmaf(f[3], a0.w, s0); s1 = fmaf(h[3], b0.w, s1);
                    s0 = fmaf(f[4], a1.x, s0); s1 = fmaf(h[4], b1.x, s1);
                    s0 = fmaf(f[5], a1.y, s0); s1 = fmaf(h[5], b1.y, s1);
                    s0 = fmaf(f[6], a1.z, s0); s1 = fmaf(h[6], b1.z, s1);
                    s0 = fmaf(f[7], a1.w, s0); s1 = fmaf(h[7], b1.w, s1);
                }
                for (; k < k_end; k += 32) {
                    float f[8];
                    ds_unpack<T>(lds128(w + 8 * k), f);
                    const float4 a0 = *reinterpret_cast<const float4*>(acts + 8 * k);
                    const float4 a1 = *reinterpret_cast<const float4*>(acts + 8 * k + 4);
                    s0 = fmaf(f[0], a0.x, s0); s0 = fmaf(f[1], a0.y, s0); s0 = fmaf(f[2], a0.z, s0); s0 = fmaf(f[3], a0.w, s0);
                    s0 = fmaf(f[4], a1.x, s0); s0 = fmaf(f[5], a1.y, s0); s0 = fmaf(f[6], a1.z, s0); s0 = fmaf(f[7], a1.w, s0);
                }
            }
            // every warp releases every chunk (the row has been read: the sums below live in registers)
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&empty_c[stage]);
            if (mine) {
                const float v = warp_sum(s0 + s1);
                if (lane == 0) red[group * kDsWarpsPerRow + wj] = v;
                named_barrier(2 + group, kDsWarpsPerRow * 32);  // the row's three warps, whatever happened
                if (wj == 0 && lane == 0 && ok) {
                    float r = 0.0f;
#pragma unroll
                    for (int q = 0; q < kDsWarpsPerRow; ++q) r += red[group * kDsWarpsPerRow + q];
                    const size_t o = (size_t)(h0 + c);
                    if (exchange) {
                        comm_put(p.comm, step, o, r);  // this rank's share of element o, to every rank
                    } else if (p.partial_out) {
                        p.partial_out[o] = r;
                    } else {
                        if (p.add_residual) r += to_float<T>(x[o]);
                        out[o] = from_float<T>(r);
                    }
                }
                named_barrier(2 + group, kDsWarpsPerRow * 32);  // `red` may be written again
            }
            if (++stage == p.rc) { stage = 0; ++use; }
            if (++turn == kDsRowGroups) turn = 0;
        }
    }
    if (!ok) atomicCAS(&p.ctl->status, 0, kStatusMoeRingConsumer);
    if (exchange) {
        named_barrier(1, kDsConsumerThreads);
        if (*(volatile int*)&s_abort == 0) {
            // one thread per output row collects the ranks' shares, in rank order
            for (int r = tid; r < n_c; r += kDsConsumerThreads) {
                const size_t o = (size_t)(h0 + r);
                float v;
                if (!comm_get_sum(p.comm, p.ctl, step, o, &v)) continue;
                if (p.add_residual) v += to_float<T>(x[o]);
                out[o] = from_float<T>(v);
            }
        }
        if (cta == 0 && tid == 0) comm_write_step(p.comm, step + 1u);  // every CTA read it at entry, before the grid barrier
    }
    if (tracer) trace_stamp(p.ctl, 5);
}

// Launches the streaming kernel when the call suits it (one token, 2-byte dtype, aligned shapes) and sets
// *handled; otherwise leaves *handled false (no error) so that the caller tries the other kernels.
int dense_ffn_stream_launch(const mk36_dense_ffn_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                            bool* handled) {
    *handled = false;
    if (a->dtype != MK36_BF16 && a->dtype != MK36_F16) return MK36_OK;
    if (a->batch != 1) return MK36_OK;
    const int H = a->hidden, I = a->intermediate;
    if (H % 8 != 0 || I % 8 != 0 || H > 8 * 4 * kDsConsumerThreads) return MK36_OK;
    const void* ptrs[] = {a->x, a->norm_weight, a->gate_weight, a->up_weight, a->down_weight};
    for (const void* q : ptrs)
        if ((reinterpret_cast<uintptr_t>(q) & 15u) != 0) return MK36_OK;
    const DeviceInfo* dev = current_device_info();
    if (!dev) return MK36_ERR_LAUNCH;
    const int ncta = dev->sm_count;
    if (H < ncta || I < ncta || (long long)H * ncta >= (1ll << 31) || (long long)I * ncta >= (1ll << 31)) return MK36_OK;
    const size_t stage_a = align_up((size_t)2 * kDsPairsPerChunk * H * 2, 128);
    const size_t stage_c = align_up((size_t)I * 2, 128);
    const size_t base_a = align_up((size_t)H * 2, 128), base_c = align_up((size_t)I * 4, 128);

    DenseStreamParams p;
    int rc = comm_params_from(comm, H, &p.comm, "dense_ffn_decode");
    if (rc != MK36_OK) return rc;
    if (p.comm.world > 1 && (!a->out || a->partial_out))
        MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: the multi-GPU entry point writes `out` and takes no partial_out");
    size_t off = 0;
    p.off_bars = (int)off;
    off += 4 * kDsMaxStages * 8;
    p.off_red = (int)off;
    off += kDsConsumerWarps * 4;
    p.off_desc = (int)off;
    off += kDsMaxStages * 8;
    off = align_up(off, 128);
    p.off_base = (int)off;
    const long long room = (long long)dev->max_smem_optin - (long long)off - 512;  // 512: the kernel's static shared memory
    long long ra = (room - (long long)base_a) / (long long)stage_a;
    long long rcn = (room - (long long)base_c) / (long long)stage_c;
    if (ra > kDsMaxStages) ra = kDsMaxStages;
    if (rcn > kDsMaxStages) rcn = kDsMaxStages;
    if (ra < 3 || rcn < 3) return MK36_OK;  // too little in flight to be worth it: the tensor-core kernel takes the call
    p.ra = (int)ra;
    p.rc = (int)rcn;
    p.stage_a_bytes = (int)stage_a;
    p.stage_c_bytes = (int)stage_c;
    p.off_ring_a = p.off_base + (int)base_a;
    p.off_ring_c = p.off_base + (int)base_c;
    const size_t end_a = (size_t)p.off_ring_a + (size_t)ra * stage_a, end_c = (size_t)p.off_ring_c + (size_t)rcn * stage_c;
    const size_t smem_bytes = end_a > end_c ? end_a : end_c;

    const size_t scratch = align_up((size_t)I * 4, 256);
    if (!workspace || reinterpret_cast<uintptr_t>(workspace) % 256 != 0)
        MK36_FAIL(MK36_ERR_WORKSPACE, "dense_ffn_decode: workspace is NULL or not 256-byte aligned");
    if (workspace_bytes < kControlBytes + scratch)
        MK36_FAIL(MK36_ERR_WORKSPACE, "dense_ffn_decode: workspace too small (%zu < %zu bytes)", workspace_bytes, kControlBytes + scratch);

    p.x = a->x;
    p.norm_w = a->norm_weight;
    p.gate = a->gate_weight;
    p.up = a->up_weight;
    p.down = a->down_weight;
    p.out = a->out;
    p.partial_out = a->partial_out;
    p.ctl = static_cast<Control*>(workspace);
    p.act = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + kControlBytes);
    p.H = H;
    p.I = I;
    p.add_residual = a->add_residual;
    p.eps = a->eps;
    p.fd_ncta = make_fastdiv(ncta);
    p.deal_static = options().moe_static ? 1 : 0;
    const void* kernel = (a->dtype == MK36_BF16) ? (const void*)dense_ffn_stream_kernel<__nv_bfloat16> : (const void*)dense_ffn_stream_kernel<__half>;
    rc = ensure_dynamic_smem(kernel, smem_bytes);
    if (rc != MK36_OK) return rc;
    void* params[] = {&p};
    rc = launch_cooperative(kernel, dim3(ncta), dim3(kDsThreads), smem_bytes, stream, params, "dense_ffn_decode(stream)");
    if (rc != MK36_OK) return rc;
    *handled = true;
    return MK36_OK;
}

}  // namespace mk36
