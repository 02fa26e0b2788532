// Library-level pieces of the C ABI: version, thread-local error text, device info cache,
// workspace initialisation / status, cooperative launch helper and the bounded-wait self test.
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <mutex>

#include "mk36_common.cuh"

namespace mk36 {

namespace {
thread_local char g_error[512] = "";
std::mutex g_info_mutex;
DeviceInfo g_info[64];
}  // namespace

Options& options() {
    static Options o;
    return o;
}

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

const DeviceInfo* current_device_info() {
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= 64) {
        set_error("cudaGetDevice failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(g_info_mutex);
    DeviceInfo& info = g_info[dev];
    if (info.device == dev) return &info;
    int sm = 0, smem = 0, coop = 0, major = 0;
    if ((e = cudaDeviceGetAttribute(&sm, cudaDevAttrMultiProcessorCount, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, dev)) != cudaSuccess ||
        (e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev)) != cudaSuccess) {
        set_error("device attribute query failed: %s", cudaGetErrorString(e));
        return nullptr;
    }
    if (major != 10) {
        set_error("this library is built for sm_100a only; device %d has compute capability %d.x", dev, major);
        return nullptr;
    }
    if (!coop) {
        set_error("device %d does not support cooperative launch", dev);
        return nullptr;
    }
    info.sm_count = sm;
    info.max_smem_optin = smem;
    info.cooperative = coop;
    info.device = dev;
    return &info;
}

int launch_cooperative(const void* kernel, dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                       void** params, const char* what) {
    cudaError_t e = cudaLaunchCooperativeKernel(kernel, grid, block, params, smem, stream);
    if (e != cudaSuccess) {
        set_error("%s: cooperative launch failed (grid %u, block %u, smem %zu): %s", what, grid.x, block.x, smem,
                  cudaGetErrorString(e));
        return MK36_ERR_LAUNCH;
    }
    return MK36_OK;
}

// Raises the kernel's dynamic shared-memory limit when a launch needs more than was set before.
// The setting is remembered per (device, kernel), so the driver call is made once, not per launch.
int ensure_dynamic_smem(const void* kernel, size_t bytes) {
    struct Entry { int device; const void* kernel; size_t bytes; };
    static thread_local Entry cache[32];
    static thread_local int used = 0;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess) dev = -1;
    for (int i = 0; i < used; ++i) {
        if (cache[i].device == dev && cache[i].kernel == kernel) {
            if (cache[i].bytes >= bytes) return MK36_OK;
            MK36_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
            cache[i].bytes = bytes;
            return MK36_OK;
        }
    }
    MK36_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    if (used < 32) cache[used++] = Entry{dev, kernel, bytes};
    return MK36_OK;
}

int max_ctas_per_sm(const void* kernel, int threads, size_t smem) {
    int n = 0;
    cudaError_t e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, threads, smem);
    if (e != cudaSuccess) {
        set_error("occupancy query failed: %s", cudaGetErrorString(e));
        return -1;
    }
    return n;
}

// Two CTAs arrive at a barrier that expects three: the wait is bound to run out.  Exercises
// the give-up path of the bounded wait without hanging anything.
__global__ void selftest_wait_kernel(Control* ctl, unsigned long long limit_ns) {
    if (threadIdx.x == 0) {
        const unsigned target = barrier_arrive(ctl, gridDim.x + 1);
        barrier_wait(ctl, target, kStatusSelfTest, limit_ns);
    }
}

}  // namespace mk36

using namespace mk36;

extern "C" {

int mk36_version(void) { return 100; }

const char* mk36_last_error(void) { return g_error; }

size_t mk36_workspace_bytes(void) { return size_t(32) << 20; }

int mk36_workspace_init(void* workspace, size_t workspace_bytes, void* stream) {
    if (!workspace) MK36_FAIL(MK36_ERR_WORKSPACE, "workspace is NULL");
    if (workspace_bytes < kControlBytes) MK36_FAIL(MK36_ERR_WORKSPACE, "workspace smaller than its control block");
    if (reinterpret_cast<uintptr_t>(workspace) % 256 != 0) MK36_FAIL(MK36_ERR_WORKSPACE, "workspace must be 256-byte aligned");
    MK36_CUDA_OK(cudaMemsetAsync(workspace, 0, kControlBytes, static_cast<cudaStream_t>(stream)));
    // the mailboxes of the MoE stream kernel, when the workspace is large enough to hold them
    if (workspace_bytes >= kTaggedEnd)
        MK36_CUDA_OK(cudaMemsetAsync(static_cast<unsigned char*>(workspace) + kMailboxOffset, 0, kTaggedEnd - kMailboxOffset, static_cast<cudaStream_t>(stream)));
    return MK36_OK;
}

int mk36_workspace_status(void* workspace, void* stream, int* device_status) {
    if (!workspace || !device_status) MK36_FAIL(MK36_ERR_INVALID_ARG, "workspace_status: NULL argument");
    Control host;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MK36_CUDA_OK(cudaMemcpyAsync(&host, workspace, sizeof(Control), cudaMemcpyDeviceToHost, s));
    MK36_CUDA_OK(cudaStreamSynchronize(s));
    *device_status = host.status;
    if (host.status != 0) MK36_FAIL(MK36_ERR_BARRIER_TIMEOUT, "a bounded device-side wait gave up (code %d)", host.status);
    return MK36_OK;
}

int mk36_set_option(const char* name, int value) {
    if (!name) MK36_FAIL(MK36_ERR_INVALID_ARG, "set_option: name is NULL");
    if (std::strcmp(name, "force_generic") == 0) {
        options().force_generic = value ? 1 : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "ring_mma") == 0) {
        options().ring_mma = value ? 1 : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "moe_stream") == 0) {
        options().moe_stream = value < 0 ? 0 : (value > 2 ? 2 : value);
        return MK36_OK;
    }
    if (std::strcmp(name, "moe_batch") == 0) {
        options().moe_batch = value ? 1 : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "moe_stages") == 0) {
        options().moe_stages = value > 0 ? value : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "static_scratch_limit") == 0) {
        options().static_scratch_limit = value > 0 ? value : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "attn_stream") == 0) {
        options().attn_stream = value ? 1 : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "dense_stream") == 0) {
        options().dense_stream = value ? 1 : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "moe_dyn_rounds") == 0) {
        options().moe_dyn_rounds = value > 0 ? value : 0;
        return MK36_OK;
    }
    if (std::strcmp(name, "linear_mma") == 0) {
        options().linear_mma = value < 0 ? 0 : value;
        return MK36_OK;
    }
    if (std::strcmp(name, "moe_static") == 0) {
        options().moe_static = value ? 1 : 0;
        return MK36_OK;
    }
    MK36_FAIL(MK36_ERR_INVALID_ARG, "set_option: unknown option '%s'", name);
}

int mk36_workspace_trace(void* workspace, void* stream, unsigned long long* stamps, int count) {
    if (!workspace || !stamps || count <= 0) MK36_FAIL(MK36_ERR_INVALID_ARG, "workspace_trace: bad argument");
    Control host;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MK36_CUDA_OK(cudaMemcpyAsync(&host, workspace, sizeof(Control), cudaMemcpyDeviceToHost, s));
    MK36_CUDA_OK(cudaStreamSynchronize(s));
    for (int i = 0; i < count; ++i) stamps[i] = i < kTraceSlots ? host.trace[i] : 0ull;
    return MK36_OK;
}

int mk36_workspace_cta_trace(void* workspace, void* stream, unsigned long long* stamps, int ctas) {
    if (!workspace || !stamps || ctas <= 0 || ctas > kCtaTraceMaxCtas) MK36_FAIL(MK36_ERR_INVALID_ARG, "workspace_cta_trace: bad argument");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    MK36_CUDA_OK(cudaMemcpyAsync(stamps, static_cast<unsigned char*>(workspace) + kCtaTraceOffset,
                                 (size_t)ctas * kCtaTraceSlots * sizeof(unsigned long long), cudaMemcpyDeviceToHost, s));
    MK36_CUDA_OK(cudaStreamSynchronize(s));
    return MK36_OK;
}

// Test hook: runs a two-CTA kernel whose barrier can never complete and whose wait gives up
// after `limit_ms`.  Afterwards mk36_workspace_status reports MK36_ERR_BARRIER_TIMEOUT and the
// workspace has to be initialised again.  No counterpart in the reference.
MK36_API int mk36_selftest_bounded_wait(void* workspace, size_t workspace_bytes, void* stream, int limit_ms) {
    if (!workspace || workspace_bytes < kControlBytes) MK36_FAIL(MK36_ERR_WORKSPACE, "selftest: bad workspace");
    if (limit_ms <= 0 || limit_ms > 2000) MK36_FAIL(MK36_ERR_INVALID_ARG, "selftest: limit_ms must be in (0, 2000]");
    selftest_wait_kernel<<<2, 32, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<Control*>(workspace),
                                                                      (unsigned long long)limit_ms * 1000000ull);
    MK36_CUDA_OK(cudaGetLastError());
    return MK36_OK;
}

}  // extern "C"
