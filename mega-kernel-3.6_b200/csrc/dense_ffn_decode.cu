// Dense SwiGLU FFN decode entry point.
//
// A dense SwiGLU FFN is the shared-expert path of the MoE layer with no routed experts, so the
// general path runs the persistent MoE kernel in its shared-only mode (experts == 0): RMSNorm ->
// gate/up rows -> one grid barrier -> down rows -> residual, weights streamed once.
// Arithmetic follows mega_kernel_qwen36/reference.py:65-88.
#include "mk36_common.cuh"

namespace mk36 {
int moe_decode_launch(const mk36_moe_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream);
int dense_ffn_mma_launch(const mk36_dense_ffn_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                         bool* handled);
int dense_ffn_stream_launch(const mk36_dense_ffn_args* a, const mk36_comm* comm, void* workspace, size_t workspace_bytes, cudaStream_t stream,
                            bool* handled);
}

using namespace mk36;

namespace {

int to_moe_args(const mk36_dense_ffn_args* a, mk36_moe_args* m) {
    if (!a) MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: args is NULL");
    if (!a->x || !a->norm_weight || !a->gate_weight || !a->up_weight || !a->down_weight)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: NULL tensor pointer");
    if (!a->out && !a->partial_out) MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: out and partial_out are both NULL");
    if (a->batch <= 0 || a->hidden <= 0 || a->intermediate <= 0)
        MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode: sizes must be positive");
    *m = mk36_moe_args{};
    m->x = a->x;
    m->norm_weight = a->norm_weight;
    m->shared_gate = a->gate_weight;
    m->shared_up = a->up_weight;
    m->shared_down = a->down_weight;
    m->out = a->out;
    m->partial_out = a->partial_out;
    m->dtype = a->dtype;
    m->batch = a->batch;
    m->hidden = a->hidden;
    m->shared_intermediate = a->intermediate;
    m->add_residual = a->add_residual;
    m->eps = a->eps;
    return MK36_OK;
}

// One token: the streaming kernel; several: the tensor-core kernel; shapes neither takes: the
// shared-expert-only mode of the MoE kernel.
int dense_launch(const mk36_dense_ffn_args* a, const mk36_moe_args* m, const mk36_comm* comm, void* workspace, size_t workspace_bytes,
                 cudaStream_t stream) {
    if (!options().force_generic) {
        bool handled = false;
        if (options().dense_stream) {
            const int rc = dense_ffn_stream_launch(a, comm, workspace, workspace_bytes, stream, &handled);
            if (rc != MK36_OK || handled) return rc;
        }
        const int rc = dense_ffn_mma_launch(a, comm, workspace, workspace_bytes, stream, &handled);
        if (rc != MK36_OK || handled) return rc;
    }
    return moe_decode_launch(m, comm, workspace, workspace_bytes, stream);
}

}  // namespace

extern "C" {

size_t mk36_dense_ffn_workspace_bytes(const mk36_dense_ffn_args* a) {
    mk36_moe_args m;
    if (to_moe_args(a, &m) != MK36_OK) return 0;
    return mk36_moe_workspace_bytes(&m);
}

int mk36_dense_ffn_decode(const mk36_dense_ffn_args* args, void* workspace, size_t workspace_bytes, void* stream) {
    mk36_moe_args m;
    int rc = to_moe_args(args, &m);
    if (rc != MK36_OK) return rc;
    return dense_launch(args, &m, nullptr, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

int mk36_dense_ffn_decode_tp(const mk36_dense_ffn_args* args, const mk36_comm* comm, void* workspace, size_t workspace_bytes,
                             void* stream) {
    if (!comm) MK36_FAIL(MK36_ERR_INVALID_ARG, "dense_ffn_decode_tp: comm is NULL");
    mk36_moe_args m;
    int rc = to_moe_args(args, &m);
    if (rc != MK36_OK) return rc;
    return dense_launch(args, &m, comm, workspace, workspace_bytes, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
