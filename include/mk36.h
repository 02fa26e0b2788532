/*
 * mk36.h - C ABI of the B200 (sm_100a) Qwen3.6 single-token decode kernels.
 *
 * One shared library (libmk36.so) exports these entry points.  They take plain device
 * pointers, sizes and a CUDA stream handle; there are no PyTorch types in any signature.  The
 * PyTorch extension `mega_kernel_qwen36._C` is a thin shim over them, and any other host
 * (ctypes, cgo, JNI, ...) can bind the same symbols.
 *
 * Conventions
 *   - every pointer in an args struct is a DEVICE pointer on the current device unless said
 *     otherwise; tensors are dense row-major ("contiguous") in the layouts named below;
 *   - `stream` is a `cudaStream_t` passed as `void*` (NULL = the legacy default stream); calls
 *     are asynchronous with respect to the host;
 *   - entry points return MK36_OK (0) or a negative mk36_status; mk36_last_error() then holds a
 *     human-readable message for the calling thread;
 *   - the decode entry points never allocate or free device memory (the one allocation the library
 *     owns is the multi-GPU exchange buffer of mk36_comm_buffer_alloc, made once at set-up).
 *     Kernels that need scratch memory or
 *     a grid-wide barrier take a caller-owned `workspace` (see mk36_workspace_*).  A workspace
 *     must not be used by two kernels that may run concurrently (use one per stream);
 *   - inputs are never written.
 *
 * Each entry point names the interface of the reference implementation
 * (MarcoDotIO/Mega-Kernel-3.6) that it replaces, as file:line within that project.
 */
#ifndef MK36_H_
#define MK36_H_

#include <stddef.h>
#include <stdint.h>

#if defined(_WIN32)
#define MK36_API __declspec(dllexport)
#else
#define MK36_API __attribute__((visibility("default")))
#endif

#ifdef __cplusplus
extern "C" {
#endif

typedef enum mk36_dtype {
    MK36_BF16 = 0,
    MK36_F16 = 1,
    MK36_F32 = 2
} mk36_dtype;

typedef enum mk36_status {
    MK36_OK = 0,
    MK36_ERR_INVALID_ARG = -1,   /* null pointer, non-positive size, inconsistent fields */
    MK36_ERR_UNSUPPORTED = -2,   /* a shape or dtype outside what the kernels handle */
    MK36_ERR_LAUNCH = -3,        /* the CUDA runtime refused a launch or a query */
    MK36_ERR_WORKSPACE = -4,     /* workspace missing, misaligned or too small */
    MK36_ERR_BARRIER_TIMEOUT = -5 /* a bounded device-side wait ran out (see workspace_status) */
} mk36_status;

/* Library version: major*10000 + minor*100 + patch. */
MK36_API int mk36_version(void);

/* Message of the last failing call made by this host thread ("" if none). */
MK36_API const char* mk36_last_error(void);

/* ---------------------------------------------------------------------------------------------
 * Workspace.  The reference allocates fresh scratch tensors with torch::empty on every call
 * (csrc/persistent_moe_decode.cu:732-745, csrc/attention_decode.cu:177-182); here the caller
 * owns one buffer per (device, stream) instead.
 *
 * mk36_workspace_bytes()       size that is enough for every op at the measured shapes
 *                              (batch <= 8 per launch); 256-byte alignment is required.
 * mk36_workspace_init()        zeroes the control block (first 32 KB: barrier counters, status
 *                              word, epoch) and, when the workspace reaches that far, the 1 MiB of
 *                              mailboxes at offset 16 MiB through which the MoE stream kernel
 *                              passes router logits between CTAs.  Must run once before first use
 *                              and after any reported timeout: a set status word is sticky, every
 *                              later kernel on the workspace leaves at once without writing its
 *                              outputs until the workspace has been initialised again.
 * mk36_workspace_status()      synchronises `stream` and returns the device status word in
 *                              *device_status: 0 = clean, otherwise the code of the bounded wait
 *                              that gave up (MK36_ERR_BARRIER_TIMEOUT is returned as well).
 * ------------------------------------------------------------------------------------------ */
MK36_API size_t mk36_workspace_bytes(void);
MK36_API int mk36_workspace_init(void* workspace, size_t workspace_bytes, void* stream);
MK36_API int mk36_workspace_status(void* workspace, void* stream, int* device_status);

/* Process-wide switches.  "force_generic" = 1 makes every op use its general register-streaming
 * kernel even where a specialised shared-memory-ring variant exists (the variants compute the same
 * function; tests use the switch to cover both).  MoE calls of one token normally run the stream
 * kernel (no grid barrier before the routing, dealt gate/up chunks) and calls of more tokens the
 * batch kernel, eight tokens per launch (one grid barrier, the same weight stream).  "moe_stream"
 * is the largest token count the stream kernel takes (default 1; 2 also sends two-token calls to
 * it, 0 none); "moe_batch" = 0 sends what the stream kernel does not take to the ring kernel
 * instead of the batch kernel; "ring_mma" = 1 additionally makes the ring kernel contract with
 * tensor-core instructions whatever the token count.  "moe_stages" (0 = default, else 2..6) sets the stream and
 * batch kernels' ring depth, "moe_static" = 1 makes them (and the dense streaming kernel) deal
 * chunks without the work counter, and "moe_dyn_rounds" (0 = default) sets how many of the last
 * rounds of gate/up chunks go through that counter; these exist for measurements.  One-token dense FFN calls normally
 * run the streaming kernel; "dense_stream" = 0 sends them to the tensor-core kernel that serves the
 * larger batches.  Attention calls with bf16 / f16 caches normally run the streaming kernel (cache
 * chunks of all KV heads through a shared-memory ring); "attn_stream" = 0 sends them to the
 * tensor-core kernel that stages the cache in registers.  "linear_mma" is the smallest token count
 * for which a projection (mk36_linear_decode) runs on tensor-core tiles (default 3, 0 = never).  Unknown names return
 * MK36_ERR_INVALID_ARG. */
MK36_API int mk36_set_option(const char* name, int value);

/* Phase trace: CTA 0 of every persistent kernel stamps the GPU's nanosecond timer at its phase
 * boundaries into the workspace (slot 0 = kernel entry).  This call synchronises `stream` and copies
 * the first `count` (<= 24) stamps of the last kernel that used the workspace to the HOST array
 * `stamps`.  The reference has no tracing beyond CUDA-event timers (benchmarks/bench_utils.py:17-56). */
MK36_API int mk36_workspace_trace(void* workspace, void* stream, unsigned long long* stamps, int count);

/* Per-CTA stamps: thread 0 of every CTA of a persistent kernel records the GPU timer at up to eight
 * phase boundaries (MoE: 0 end of routed gate/up, 1 after the grid barrier, 2 end of down rows, 3 entry,
 * 4 logits published).  Copies 8 stamps for each of the first `ctas` (<= 192) CTAs to the HOST array
 * `stamps` [ctas][8] after synchronising `stream`; the spread across CTAs shows load imbalance. */
MK36_API int mk36_workspace_cta_trace(void* workspace, void* stream, unsigned long long* stamps, int ctas);

/* Test hook for the give-up path of the bounded device-side waits: launches two CTAs whose barrier
 * expects a third arrival that never comes; each wait returns after `limit_ms` (1..2000) and
 * records its code in the status word, so that mk36_workspace_status then reports
 * MK36_ERR_BARRIER_TIMEOUT.  Nothing hangs or faults; the workspace must be initialised again
 * afterwards.  No counterpart in the reference (its grid.sync() calls are unbounded:
 * csrc/persistent_moe_decode.cu:517-564). */
MK36_API int mk36_selftest_bounded_wait(void* workspace, size_t workspace_bytes, void* stream, int limit_ms);

/* ---------------------------------------------------------------------------------------------
 * MoE decode: RMSNorm -> router logits -> top-k -> softmax over the k survivors -> routed
 * SwiGLU experts + shared SwiGLU expert -> down projections -> (+ residual).
 *
 * Replaces `moe_decode_persistent_cuda` (csrc/persistent_moe_decode.cu:701-860, bound at
 * csrc/bindings.cpp:33) and the grouped torch path `_moe_decode_grouped_torch`
 * (mega_kernel_qwen36/ops.py:161-199); results follow `moe_decode_reference`
 * (mega_kernel_qwen36/reference.py:16-62), including the rounding of the normalised input to
 * the activation dtype before the projections.
 *
 * Layouts: x [batch, hidden]; norm_weight [hidden]; router_weight [experts, hidden];
 * expert_gate, expert_up [local_experts, intermediate, hidden];
 * expert_down [local_experts, hidden, intermediate]; shared_gate, shared_up
 * [shared_intermediate, hidden]; shared_down [hidden, shared_intermediate];
 * out [batch, hidden] (same dtype as x); indices [batch, top_k] int64, sorted by descending
 * logit; route_weights [batch, top_k] fp32.
 *
 * Expert parallelism: a rank that holds experts [expert_base, expert_base + local_experts)
 * passes only those slabs; routing is still computed over all `experts` router rows, and only
 * the selected experts that are local contribute.  With partial_out != NULL the kernel writes
 * the fp32 partial sum [batch, hidden] (no residual, no rounding) there instead of `out`
 * (out may then be NULL); the caller reduces the partials across ranks and adds the residual.
 * The shared expert is split by passing a slice of its intermediate rows/columns.
 * Single-GPU callers set expert_base = 0, local_experts = experts, partial_out = NULL.
 *
 * experts == 0 && top_k == 0 runs the shared path only (that is a dense SwiGLU FFN).
 * ------------------------------------------------------------------------------------------ */
typedef struct mk36_moe_args {
    const void* x;
    const void* norm_weight;
    const void* router_weight;
    const void* expert_gate;
    const void* expert_up;
    const void* expert_down;
    const void* shared_gate;
    const void* shared_up;
    const void* shared_down;
    void* out;
    int64_t* indices;
    float* route_weights;
    float* partial_out;
    int32_t dtype; /* mk36_dtype of x, every weight and out */
    int32_t batch;
    int32_t hidden;
    int32_t experts;
    int32_t top_k;
    int32_t intermediate;
    int32_t shared_intermediate;
    int32_t expert_base;
    int32_t local_experts;
    int32_t add_residual;
    float eps;
} mk36_moe_args;

MK36_API size_t mk36_moe_workspace_bytes(const mk36_moe_args* args);
MK36_API int mk36_moe_decode(const mk36_moe_args* args, void* workspace, size_t workspace_bytes,
                             void* stream);

/* ---------------------------------------------------------------------------------------------
 * Dense SwiGLU FFN decode: RMSNorm -> silu(x Wg^T) * (x Wu^T) -> Wd -> (+ residual).
 *
 * The reference has no native kernel for this op; this replaces `_dense_ffn_decode_torch`
 * (mega_kernel_qwen36/ops.py:202-218) and `dense_ffn_decode_triton`
 * (mega_kernel_qwen36/triton_ops.py:94-109); results follow `dense_ffn_decode_reference`
 * (mega_kernel_qwen36/reference.py:65-88).
 *
 * Layouts: x [batch, hidden]; norm_weight [hidden]; gate_weight, up_weight
 * [intermediate, hidden]; down_weight [hidden, intermediate]; out [batch, hidden].
 *
 * Tensor parallelism: a rank passes its row slice of gate/up and the matching column slice of
 * down stored densely as [hidden, intermediate_local]; with partial_out != NULL the fp32 partial
 * [batch, hidden] is written (no residual) for the caller's all-reduce.
 * ------------------------------------------------------------------------------------------ */
typedef struct mk36_dense_ffn_args {
    const void* x;
    const void* norm_weight;
    const void* gate_weight;
    const void* up_weight;
    const void* down_weight;
    void* out;
    float* partial_out;
    int32_t dtype;
    int32_t batch;
    int32_t hidden;
    int32_t intermediate;
    int32_t add_residual;
    float eps;
} mk36_dense_ffn_args;

MK36_API size_t mk36_dense_ffn_workspace_bytes(const mk36_dense_ffn_args* args);
MK36_API int mk36_dense_ffn_decode(const mk36_dense_ffn_args* args, void* workspace,
                                   size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Full-attention GQA decode of one query token over an existing KV cache (soft-max over the
 * whole cache, no causal mask): out[b,h,:] = softmax(scale * q[b,h,:] . K[b,:,h/g,:]) V[b,:,h/g,:].
 *
 * Replaces `full_attention_decode_cuda` (csrc/attention_decode.cu:152-218, bound at
 * csrc/bindings.cpp:34); results follow `full_attention_decode_reference`
 * (mega_kernel_qwen36/reference.py:117-145).
 *
 * Layouts: q, out [batch, query_heads, head_dim]; k_cache, v_cache
 * [batch, seq_len, kv_heads, head_dim].  query_heads % kv_heads == 0, head_dim <= 256,
 * seq_len > 0.  KV-head parallel ranks simply pass their own head slices.
 * ------------------------------------------------------------------------------------------ */
typedef struct mk36_attention_args {
    const void* q;
    const void* k_cache;
    const void* v_cache;
    void* out;
    int32_t dtype;
    int32_t batch;
    int32_t query_heads;
    int32_t kv_heads;
    int32_t head_dim;
    int32_t seq_len;
    float scale;
} mk36_attention_args;

MK36_API size_t mk36_attention_workspace_bytes(const mk36_attention_args* args);
MK36_API int mk36_full_attention_decode(const mk36_attention_args* args, void* workspace,
                                        size_t workspace_bytes, void* stream);

/* Full-attention decode for callers that cannot provide a workspace.  This entry point has no
 * counterpart in the reference: it exists for hosts that bind the library over a plain C boundary
 * and own no device allocator, or that sit in a request loop where cudaMalloc / cudaFree (which
 * synchronise the device) must not be called.  Same arithmetic, same kernels and same results as
 * mk36_full_attention_decode (bit-identical whenever both pick the same kernel, which they do when the
 * streaming kernel's partial rows fit the array); the split partials and the barrier control block live in a fixed
 * MK36_STATIC_SCRATCH_BYTES device array inside the library, and the call performs no device
 * allocation of any kind.
 *   - A problem whose launch plan needs more scratch than the array holds fails with
 *     MK36_ERR_WORKSPACE and a message that names the limit, before anything is launched (`out` is
 *     left untouched).  With bf16 / f16 inputs, head_dim 64 / 128 / 256 and up to 8 query heads per KV
 *     head the need is one partial row (head_dim + 2 floats) per query head and SM: 2.5 MB for 16
 *     heads of 256 on a 148-SM part; when the streaming kernel's rows do not fit, the call takes the
 *     register-staged tensor-core kernel with half as many rows or fewer.  Other dtypes and head sizes
 *     take the general kernel, whose need grows with its occupancy and can exceed the array.
 *   - All calls on one GPU share the array.  Each call clears the control block on `stream` before
 *     its kernels; calls that may overlap on the same GPU (other streams or host threads) race on
 *     the array and their results are undefined - serialise them.
 *   - The first call on each GPU also looks up the array's device address; make that first call
 *     outside of any stream capture.
 *   - The bounded device-side wait of the attention kernels records a give-up in a status word that
 *     lives in the array.  mk36_static_scratch_status synchronises `stream` and returns that word in
 *     *device_status (0 = clean; otherwise the code, and MK36_ERR_BARRIER_TIMEOUT as the return
 *     value); call it before the next static call on the GPU, which clears the word.  A call whose
 *     status is not 0 may have left `out` partly unwritten.
 * mk36_set_option("static_scratch_limit", n) makes the entry point treat its array as n bytes
 * (0 = the full size), so that the refusal can be tried with a small problem. */
#define MK36_STATIC_SCRATCH_BYTES (4u << 20)
MK36_API int mk36_full_attention_decode_static(const mk36_attention_args* args, void* stream);
MK36_API int mk36_static_scratch_status(void* stream, int* device_status);

/* ---------------------------------------------------------------------------------------------
 * Linear-attention recurrent decode step with an fp32 state:
 *     S'[b,h] = decay * S[b,h] + k[b,hk] (x) (beta * v[b,h]);   out[b,h] = q[b,hk]^T S'[b,h]
 *
 * Replaces `linear_attention_decode_cuda` (csrc/linear_attention_decode.cu:46-93, bound at
 * csrc/bindings.cpp:35); results follow `linear_attention_decode_reference`
 * (mega_kernel_qwen36/reference.py:148-166): scalar decay, no beta, equal head counts.
 *
 * Layouts: q, k [batch, key_heads, key_dim]; v, out [batch, value_heads, value_dim];
 * state, new_state [batch, value_heads, key_dim, value_dim] fp32.  value_heads must be a
 * multiple of key_heads (key head h / (value_heads / key_heads) serves value head h).
 * new_state may equal state (in-place update); otherwise state is left untouched.
 * decay_per_head / beta_per_head, when non-NULL, are fp32 [batch, value_heads] and override
 * the scalar `decay` / a beta of 1.  No workspace is needed.
 * ------------------------------------------------------------------------------------------ */
typedef struct mk36_linear_attention_args {
    const void* q;
    const void* k;
    const void* v;
    const float* state;
    void* out;
    float* new_state;
    const float* decay_per_head;
    const float* beta_per_head;
    int32_t dtype; /* of q, k, v, out */
    int32_t batch;
    int32_t key_heads;
    int32_t value_heads;
    int32_t key_dim;
    int32_t value_dim;
    float decay;
} mk36_linear_attention_args;

MK36_API int mk36_linear_attention_decode(const mk36_linear_attention_args* args, void* stream);

/* Several consecutive steps of the same recurrence in one call, the fp32 state resident on chip:
 * q, k are [steps, batch, key_heads, key_dim], v and out [steps, batch, value_heads, value_dim];
 * step t reads its q/k/v, updates the state and writes out[t]; the state is read from `state` once and
 * written to `new_state` once (they may be the same buffer).  decay_per_step / beta_per_step are
 * optional fp32 [steps, batch, value_heads] gates (NULL: the scalar `decay`, beta 1).  Outputs
 * and final state are bit-identical to `steps` calls of mk36_linear_attention_decode.  The reference's
 * operator is one step per call (mega_kernel_qwen36/ops.py:377-386), so this entry point has no
 * counterpart there; it exists because a one-step call has to move the whole state (2 MiB per
 * batch row at the 35B-A3B shape) through HBM twice per token. */
typedef struct mk36_linear_attention_steps_args {
    const void* q;
    const void* k;
    const void* v;
    const float* state;
    void* out;
    float* new_state;
    const float* decay_per_step;
    const float* beta_per_step;
    int32_t dtype; /* of q, k, v, out */
    int32_t steps;
    int32_t batch;
    int32_t key_heads;
    int32_t value_heads;
    int32_t key_dim;
    int32_t value_dim;
    float decay;
} mk36_linear_attention_steps_args;

MK36_API int mk36_linear_attention_decode_steps(const mk36_linear_attention_steps_args* args, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Decode-time projection of one to eight tokens:
 *     out[b, :] = weight . xin[b, :] (+ residual[b, :]),   xin = RMSNorm(x; norm_weight, eps) or x,
 * with an optional arg-max over each output row.
 *
 * No counterpart among the reference's kernels: these are the `linear` (q/k/v projection),
 * `linear_residual` (attention output projection plus residual) and `lm_head` / arg-max tasks that
 * the reference's decode task graph names (mega_kernel_qwen36/mpk_graph.py:352-398, 418-427,
 * 496-514) and leaves to the caller, whose decode layer takes q, k and v as inputs
 * (mega_kernel_qwen36/ops.py:701-748).  Arithmetic as everywhere else in the reference: RMSNorm in
 * fp32 with the result rounded to the tensors' dtype (mega_kernel_qwen36/reference.py:10-13), fp32
 * accumulation, one rounding after the residual was added.
 *
 * Layouts: x [batch, in_features]; weight [out_features, in_features] (torch.nn.functional.linear);
 * norm_weight [in_features] or NULL; residual [batch, out_features] or NULL; out
 * [batch, out_features]; argmax int64 [batch] or NULL: the index of the largest value of the stored
 * (rounded) output row, the lowest index among equals.  bf16 / f16; batch <= 8; in_features a
 * multiple of 8, at most 16384, and batch x in_features x 2 bytes at most 64 KB (a count of three or
 * five to seven tokens is padded to the next multiple of four for that bound).  Other shapes return
 * MK36_ERR_UNSUPPORTED.  The workspace is used for its control block only (status word, arg-max
 * slots): mk36_linear_workspace_bytes() bytes, initialised like every workspace.
 * ------------------------------------------------------------------------------------------ */
typedef struct mk36_linear_args {
    const void* x;
    const void* norm_weight;
    const void* weight;
    const void* residual;
    void* out;
    int64_t* argmax;
    int32_t dtype;
    int32_t batch;
    int32_t in_features;
    int32_t out_features;
    float eps;
} mk36_linear_args;

MK36_API size_t mk36_linear_workspace_bytes(const mk36_linear_args* args);
MK36_API int mk36_linear_decode(const mk36_linear_args* args, void* workspace, size_t workspace_bytes, void* stream);

/* ---------------------------------------------------------------------------------------------
 * Multi-GPU (one process per GPU, all GPUs on one NVLink / NVSwitch box).
 *
 * The reference is single-GPU; these entry points have no counterpart there.  They run the same
 * kernels as mk36_moe_decode / mk36_dense_ffn_decode on the rank's shard of the weights
 * (expert-parallel MoE: experts [expert_base, expert_base + local_experts) plus this rank's slice
 * of the shared expert's intermediate rows; tensor-parallel dense FFN: this rank's gate/up rows and
 * down columns) and finish, inside the same launch, with the sum of all ranks' fp32 partial outputs
 * over peer memory, the residual and the rounding.  Every rank ends with the same, bit-identical,
 * full `out`; `partial_out` must be NULL.
 *
 * Each rank owns one exchange buffer of mk36_comm_buffer_bytes() bytes from mk36_comm_buffer_alloc
 * (a plain cudaMalloc, zero-filled: CUDA IPC can export nothing smaller than a whole allocation;
 * this is the only device memory the library allocates, once at set-up).  The ranks swap
 * mk36_ipc_export handles by any host channel, map the others' buffers with mk36_ipc_open, and
 * describe the result in mk36_comm (buffers[rank] is the rank's own pointer).  All ranks must make
 * the same sequence of *_ep / *_tp calls with the same shapes.  A device-side wait for a peer is
 * bounded (about a second); when it runs out the status word of the workspace is set to 401 and
 * the kernel ends. */
#define MK36_MAX_RANKS 8
#define MK36_IPC_HANDLE_BYTES 64

typedef struct mk36_comm {
    int32_t rank;
    int32_t world;
    void* buffers[MK36_MAX_RANKS];
} mk36_comm;

MK36_API size_t mk36_comm_buffer_bytes(void);
MK36_API int mk36_comm_buffer_alloc(void** buffer);
/* Clears the rank's OWN buffer (step counter, slots) on `stream`: the way back after a step in which a rank gave up
 * on a peer (status 401), which leaves the ranks' step counters in disagreement.  Every rank calls it, with a host
 * barrier before and after; workspaces whose status was set need mk36_workspace_init as well. */
MK36_API int mk36_comm_buffer_reset(void* buffer, void* stream);
MK36_API int mk36_comm_buffer_free(void* buffer);
MK36_API int mk36_ipc_export(void* buffer, unsigned char handle[MK36_IPC_HANDLE_BYTES]);
MK36_API int mk36_ipc_open(const unsigned char handle[MK36_IPC_HANDLE_BYTES], void** buffer);
MK36_API int mk36_ipc_close(void* buffer);
MK36_API int mk36_moe_decode_ep(const mk36_moe_args* args, const mk36_comm* comm, void* workspace,
                                size_t workspace_bytes, void* stream);
MK36_API int mk36_dense_ffn_decode_tp(const mk36_dense_ffn_args* args, const mk36_comm* comm, void* workspace,
                                      size_t workspace_bytes, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MK36_H_ */
