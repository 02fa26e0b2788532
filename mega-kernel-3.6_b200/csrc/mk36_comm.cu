// Host side of the cross-GPU exchange buffers: allocation, CUDA IPC export / import, and the
// translation of the C-ABI descriptor into kernel parameters.
//
// The exchange buffer is the one piece of device memory this library allocates itself: CUDA IPC
// exports whole cudaMalloc allocations, and a pointer carved out of a framework's caching
// allocator cannot be exported reliably.  It is allocated once per rank at set-up, never on the
// decode path.
#include <cstring>

#include "mk36_comm.cuh"

namespace mk36 {

int comm_params_from(const mk36_comm* c, int hidden, CommParams* out, const char* what) {
    *out = CommParams{};
    if (!c || c->world <= 1) return MK36_OK;
    if (c->world > kCommMaxRanks) MK36_FAIL(MK36_ERR_UNSUPPORTED, "%s: world size %d exceeds %d", what, c->world, kCommMaxRanks);
    if (c->rank < 0 || c->rank >= c->world) MK36_FAIL(MK36_ERR_INVALID_ARG, "%s: rank %d outside [0, %d)", what, c->rank, c->world);
    if ((size_t)hidden * 8 > (size_t)kCommMaxElems)
        MK36_FAIL(MK36_ERR_UNSUPPORTED, "%s: hidden %d exceeds the exchange buffer's %d values per token", what, hidden, kCommMaxElems / 8);
    out->rank = c->rank;
    out->world = c->world;
    for (int q = 0; q < c->world; ++q) {
        if (!c->buffers[q] || reinterpret_cast<uintptr_t>(c->buffers[q]) % 256 != 0)
            MK36_FAIL(MK36_ERR_INVALID_ARG, "%s: exchange buffer of rank %d is NULL or not 256-byte aligned", what, q);
        out->buf[q] = static_cast<unsigned char*>(c->buffers[q]);
    }
    return MK36_OK;
}

}  // namespace mk36

using namespace mk36;

extern "C" {

size_t mk36_comm_buffer_bytes(void) { return kCommBytes; }

int mk36_comm_buffer_alloc(void** buffer) {
    if (!buffer) MK36_FAIL(MK36_ERR_INVALID_ARG, "comm_buffer_alloc: buffer is NULL");
    void* p = nullptr;
    MK36_CUDA_OK(cudaMalloc(&p, kCommBytes));
    cudaError_t e = cudaMemset(p, 0, kCommBytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        cudaFree(p);
        MK36_FAIL(MK36_ERR_LAUNCH, "comm_buffer_alloc: clearing the buffer failed: %s", cudaGetErrorString(e));
    }
    *buffer = p;
    return MK36_OK;
}

// Puts the rank's own buffer back into the state mk36_comm_buffer_alloc left it in (step counter and every slot
// zero), on `stream`.  After a step in which a rank gave up on a peer the ranks' step counters disagree for good;
// this is the way back without a new allocation and a new IPC exchange.  Collective in spirit: every rank resets
// its own buffer, with a host barrier before (no rank is still inside a step) and after (nobody starts the next
// step against a buffer that is not clear yet); the workspaces whose status was set need mk36_workspace_init too.
int mk36_comm_buffer_reset(void* buffer, void* stream) {
    if (!buffer) MK36_FAIL(MK36_ERR_INVALID_ARG, "comm_buffer_reset: buffer is NULL");
    MK36_CUDA_OK(cudaMemsetAsync(buffer, 0, kCommBytes, static_cast<cudaStream_t>(stream)));
    return MK36_OK;
}

int mk36_comm_buffer_free(void* buffer) {
    if (buffer) MK36_CUDA_OK(cudaFree(buffer));
    return MK36_OK;
}

int mk36_ipc_export(void* buffer, unsigned char handle[MK36_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == MK36_IPC_HANDLE_BYTES, "IPC handle size");
    if (!buffer || !handle) MK36_FAIL(MK36_ERR_INVALID_ARG, "ipc_export: NULL argument");
    cudaIpcMemHandle_t h;
    MK36_CUDA_OK(cudaIpcGetMemHandle(&h, buffer));
    std::memcpy(handle, &h, sizeof(h));
    return MK36_OK;
}

int mk36_ipc_open(const unsigned char handle[MK36_IPC_HANDLE_BYTES], void** buffer) {
    if (!buffer || !handle) MK36_FAIL(MK36_ERR_INVALID_ARG, "ipc_open: NULL argument");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* p = nullptr;
    MK36_CUDA_OK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *buffer = p;
    return MK36_OK;
}

int mk36_ipc_close(void* buffer) {
    if (buffer) MK36_CUDA_OK(cudaIpcCloseMemHandle(buffer));
    return MK36_OK;
}

}  // extern "C"
