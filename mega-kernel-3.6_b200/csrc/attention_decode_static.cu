// Full-attention decode without a caller-owned workspace.
//
// Who this is for: hosts that reach the library through a plain foreign-function boundary (a
// ctypes / cgo / JNI shim, an inference server's plugin slot) and have no device allocator of
// their own to carve a workspace from, or that run inside a request loop where calling
// cudaMalloc / cudaFree is off the table because those calls synchronise the whole device and
// stall every other stream.  Such a caller can hand over its input and output tensors, but it
// cannot create the scratch buffer that mk36_full_attention_decode asks for.
//
// mk36_full_attention_decode_static runs the same kernels as mk36_full_attention_decode, with the
// split-KV partials and the grid-barrier control block placed in the fixed device array below
// instead of a workspace argument.  It never calls cudaMalloc, cudaFree or any allocating library
// routine.  Consequences of the fixed array, all part of the contract:
//   * every GPU that loads the library carries the array (kStaticScratchBytes) until the process
//     exits, whether or not the entry point is ever called;
//   * problems whose partials do not fit are rejected with MK36_ERR_WORKSPACE and a message that
//     names the limit, before anything is launched (the output is left untouched); use the
//     workspace variant for those;
//   * all calls on one GPU share the array and it keeps whatever the previous call left in it.
//     The control block is therefore cleared (cudaMemsetAsync on the caller's stream) at the
//     start of every call; the partials need no clearing because each call overwrites every slot it
//     later reads.  Two calls whose kernels may overlap on the same GPU (different streams,
//     different host threads) race on the array and give undefined results - serialise them;
//   * the first call on each GPU looks up the array's device address (cudaGetSymbolAddress, once
//     per device, with that device current).  Make that first call before any stream capture;
//   * a bounded device-side wait that gave up leaves its code in the array's status word, where the
//     caller has no pointer to look: mk36_static_scratch_status reads it.  Ask before the next static
//     call on that GPU, because that call clears the word again.
//
// The array's name is only a host-side handle in host code; the kernels get the device address
// obtained below.
#include <mutex>

#include "mk36_common.cuh"

namespace mk36 {

int attention_decode_launch(const mk36_attention_args* a, void* workspace, size_t workspace_bytes, cudaStream_t stream);

namespace {

// Control block + split-KV partials.  A launch holds one partial row (head_dim + 2 floats) per
// (batch item, query head, split).  The streaming kernel runs one CTA per SM over all KV heads, so with
// bf16 / f16 inputs, head_dim 64 / 128 / 256 and up to 8 query heads per KV head the need is one row per
// query head and SM (2.5 MB for 16 heads of 256 on a 148-SM part); when that does not fit, the
// register-staged tensor-core kernel with at most half as many rows takes the call.  The general kernel (other dtypes and head sizes) runs several CTAs per SM with up to
// four heads each, and its need depends on that occupancy; it can exceed the array.  Either way the
// launcher compares the exact need of every launch of the call with this size before it launches
// anything and refuses the call when one does not fit.
constexpr size_t kStaticScratchBytes = MK36_STATIC_SCRATCH_BYTES;

static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mutex;
void* g_static_ptr[kMaxDevices] = {};

// Device address of the scratch array on the current device; looked up once per device.
int static_scratch_for_current_device(void** out) {
    int dev = -1;
    MK36_CUDA_OK(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) MK36_FAIL(MK36_ERR_LAUNCH, "full_attention_decode_static: device index %d out of range", dev);
    std::lock_guard<std::mutex> lock(g_static_mutex);
    if (!g_static_ptr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_scratch);
        if (e != cudaSuccess || !ptr) {
            set_error("full_attention_decode_static: cudaGetSymbolAddress failed on device %d: %s", dev, cudaGetErrorString(e));
            return MK36_ERR_LAUNCH;
        }
        g_static_ptr[dev] = ptr;
    }
    *out = g_static_ptr[dev];
    return MK36_OK;
}

}  // namespace
}  // namespace mk36

using namespace mk36;

extern "C" {

int mk36_full_attention_decode_static(const mk36_attention_args* args, void* stream) {
    if (!args) MK36_FAIL(MK36_ERR_INVALID_ARG, "full_attention_decode_static: args is NULL");
    void* scratch = nullptr;
    int rc = static_scratch_for_current_device(&scratch);
    if (rc != MK36_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // start from a clean control block: the previous call may have been abandoned half way
    MK36_CUDA_OK(cudaMemsetAsync(scratch, 0, kControlBytes, s));
    // the launcher checks every launch's exact scratch need against the size given here ("static_scratch_limit"
    // lets a test lower it so that the refusal can be exercised with a small problem)
    size_t limit = kStaticScratchBytes;
    if (options().static_scratch_limit > 0 && (size_t)options().static_scratch_limit < limit) limit = (size_t)options().static_scratch_limit;
    rc = attention_decode_launch(args, scratch, limit, s);
    if (rc == MK36_ERR_WORKSPACE) {
        MK36_FAIL(MK36_ERR_WORKSPACE,
                  "full_attention_decode_static: batch %d x %d query heads x head_dim %d at %d cached tokens needs more scratch than the "
                  "built-in %zu-byte buffer; call mk36_full_attention_decode with a caller-owned workspace instead",
                  args->batch, args->query_heads, args->head_dim, args->seq_len, limit);
    }
    return rc;
}

int mk36_static_scratch_status(void* stream, int* device_status) {
    if (!device_status) MK36_FAIL(MK36_ERR_INVALID_ARG, "static_scratch_status: device_status is NULL");
    void* scratch = nullptr;
    const int rc = static_scratch_for_current_device(&scratch);
    if (rc != MK36_OK) return rc;
    return mk36_workspace_status(scratch, stream, device_status);
}

}  // extern "C"
