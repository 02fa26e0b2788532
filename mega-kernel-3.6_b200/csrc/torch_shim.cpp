// PyTorch extension `mega_kernel_qwen36._C`: a thin shim over the C ABI in include/mk36.h.
//
// It exports the three functions the reference's pybind module exports
// (csrc/bindings.cpp:32-36: moe_decode_persistent, full_attention_decode,
// linear_attention_decode) with the same signatures, plus dense_ffn_decode and the
// expert-/tensor-parallel and per-head variants.  The shim validates tensors (same messages as
// the reference's TORCH_CHECKs), allocates outputs, owns one workspace per device and passes raw
// pointers and the current stream to libmk36; it contains no kernels and no arithmetic.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include <map>
#include <mutex>
#include <optional>
#include <tuple>

#include "mk36.h"

namespace {

#define SHIM_CHECK_CUDA(x) TORCH_CHECK((x).is_cuda(), #x " must be a CUDA tensor")
#define SHIM_CHECK_CONTIGUOUS(x) TORCH_CHECK((x).is_contiguous(), #x " must be contiguous")
#define SHIM_CHECK_INPUT(x) \
    SHIM_CHECK_CUDA(x);     \
    SHIM_CHECK_CONTIGUOUS(x)

int dtype_code(const torch::Tensor& t, const char* what) {
    switch (t.scalar_type()) {
        case at::ScalarType::BFloat16: return MK36_BF16;
        case at::ScalarType::Half: return MK36_F16;
        case at::ScalarType::Float: return MK36_F32;
        default: TORCH_CHECK(false, what, ": dtype ", t.scalar_type(), " is not supported (bfloat16, float16, float32)");
    }
    return -1;
}

void check_rc(int rc) { TORCH_CHECK(rc == MK36_OK, mk36_last_error(), " (mk36 status ", rc, ")"); }

// One workspace per device, grown on demand, initialised once.  Kernels that share it are
// ordered by the stream they run on; callers that launch on several streams of one device at the
// same time must serialise those launches.
struct Workspace {
    torch::Tensor buffer;
    size_t bytes = 0;
};
std::mutex g_ws_mutex;
std::map<int, Workspace> g_workspaces;

Workspace& workspace_for(const torch::Tensor& like, size_t need) {
    std::lock_guard<std::mutex> lock(g_ws_mutex);
    Workspace& ws = g_workspaces[like.get_device()];
    size_t want = mk36_workspace_bytes();
    if (need > want) want = need;
    if (ws.bytes < want) {
        // Run each op once eagerly before capturing it in a CUDA graph, so that this allocation
        // and its initialisation happen outside the capture.
        ws.buffer = torch::empty({static_cast<int64_t>(want)}, like.options().dtype(torch::kUInt8));
        ws.bytes = want;
        check_rc(mk36_workspace_init(ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    }
    return ws;
}

void check_moe_tensors(const torch::Tensor& x, const torch::Tensor& norm_weight, const torch::Tensor& router_weight,
                       const torch::Tensor& expert_gate, const torch::Tensor& expert_up, const torch::Tensor& expert_down,
                       const torch::Tensor& shared_gate, const torch::Tensor& shared_up, const torch::Tensor& shared_down,
                       int64_t top_k, int64_t local_experts) {
    SHIM_CHECK_INPUT(x);
    SHIM_CHECK_INPUT(norm_weight);
    SHIM_CHECK_INPUT(router_weight);
    SHIM_CHECK_INPUT(expert_gate);
    SHIM_CHECK_INPUT(expert_up);
    SHIM_CHECK_INPUT(expert_down);
    SHIM_CHECK_INPUT(shared_gate);
    SHIM_CHECK_INPUT(shared_up);
    SHIM_CHECK_INPUT(shared_down);
    TORCH_CHECK(x.dim() == 2, "x must be [batch, hidden]");
    TORCH_CHECK(norm_weight.dim() == 1, "norm_weight must be [hidden]");
    TORCH_CHECK(router_weight.dim() == 2, "router_weight must be [experts, hidden]");
    TORCH_CHECK(expert_gate.dim() == 3, "expert_gate must be [experts, intermediate, hidden]");
    TORCH_CHECK(expert_up.sizes() == expert_gate.sizes(), "expert_up shape must match expert_gate");
    TORCH_CHECK(expert_down.dim() == 3, "expert_down must be [experts, hidden, intermediate]");
    TORCH_CHECK(shared_gate.dim() == 2, "shared_gate must be [shared_intermediate, hidden]");
    TORCH_CHECK(shared_up.sizes() == shared_gate.sizes(), "shared_up shape must match shared_gate");
    TORCH_CHECK(shared_down.dim() == 2, "shared_down must be [hidden, shared_intermediate]");
    const auto dt = x.scalar_type();
    TORCH_CHECK(dt == norm_weight.scalar_type(), "x and norm_weight dtype mismatch");
    TORCH_CHECK(dt == router_weight.scalar_type(), "x and router_weight dtype mismatch");
    TORCH_CHECK(dt == expert_gate.scalar_type(), "x and expert_gate dtype mismatch");
    TORCH_CHECK(dt == expert_up.scalar_type(), "x and expert_up dtype mismatch");
    TORCH_CHECK(dt == expert_down.scalar_type(), "x and expert_down dtype mismatch");
    TORCH_CHECK(dt == shared_gate.scalar_type(), "x and shared_gate dtype mismatch");
    TORCH_CHECK(dt == shared_up.scalar_type(), "x and shared_up dtype mismatch");
    TORCH_CHECK(dt == shared_down.scalar_type(), "x and shared_down dtype mismatch");
    const int64_t hidden = x.size(1);
    const int64_t experts = router_weight.size(0);
    const int64_t intermediate = expert_gate.size(1);
    const int64_t shared_intermediate = shared_gate.size(0);
    TORCH_CHECK(top_k > 0 && top_k <= experts, "top_k must be in [1, experts]");
    TORCH_CHECK(norm_weight.size(0) == hidden, "norm_weight hidden mismatch");
    TORCH_CHECK(router_weight.size(1) == hidden, "router_weight hidden mismatch");
    TORCH_CHECK(expert_gate.size(0) == local_experts && expert_gate.size(2) == hidden, "expert_gate shape mismatch");
    TORCH_CHECK(expert_down.size(0) == local_experts && expert_down.size(1) == hidden && expert_down.size(2) == intermediate,
                "expert_down shape mismatch");
    TORCH_CHECK(shared_gate.size(1) == hidden, "shared_gate hidden mismatch");
    TORCH_CHECK(shared_down.size(0) == hidden && shared_down.size(1) == shared_intermediate, "shared_down shape mismatch");
}

mk36_moe_args moe_args(const torch::Tensor& x, const torch::Tensor& norm_weight, const torch::Tensor& router_weight,
                       const torch::Tensor& expert_gate, const torch::Tensor& expert_up, const torch::Tensor& expert_down,
                       const torch::Tensor& shared_gate, const torch::Tensor& shared_up, const torch::Tensor& shared_down,
                       double eps, int64_t top_k, bool add_residual) {
    mk36_moe_args a{};
    a.x = x.data_ptr();
    a.norm_weight = norm_weight.data_ptr();
    a.router_weight = router_weight.data_ptr();
    a.expert_gate = expert_gate.data_ptr();
    a.expert_up = expert_up.data_ptr();
    a.expert_down = expert_down.data_ptr();
    a.shared_gate = shared_gate.data_ptr();
    a.shared_up = shared_up.data_ptr();
    a.shared_down = shared_down.data_ptr();
    a.dtype = dtype_code(x, "moe_decode");
    a.batch = static_cast<int32_t>(x.size(0));
    a.hidden = static_cast<int32_t>(x.size(1));
    a.experts = static_cast<int32_t>(router_weight.size(0));
    a.top_k = static_cast<int32_t>(top_k);
    a.intermediate = static_cast<int32_t>(expert_gate.size(1));
    a.shared_intermediate = static_cast<int32_t>(shared_gate.size(0));
    a.expert_base = 0;
    a.local_experts = a.experts;
    a.add_residual = add_residual ? 1 : 0;
    a.eps = static_cast<float>(eps);
    return a;
}

// -------------------------------------------------------------------------------------------
// moe_decode_persistent: same name, arguments and return value as csrc/bindings.cpp:33.
// -------------------------------------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> moe_decode_persistent(
    torch::Tensor x, torch::Tensor norm_weight, torch::Tensor router_weight, torch::Tensor expert_gate, torch::Tensor expert_up,
    torch::Tensor expert_down, torch::Tensor shared_gate, torch::Tensor shared_up, torch::Tensor shared_down, double eps,
    int64_t top_k, bool add_residual) {
    check_moe_tensors(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down,
                      top_k, router_weight.size(0));
    const c10::cuda::CUDAGuard guard(x.device());
    mk36_moe_args a =
        moe_args(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down, eps,
                 top_k, add_residual);
    auto out = torch::empty_like(x);
    auto indices = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kInt64));
    auto weights = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kFloat32));
    a.out = out.data_ptr();
    a.indices = indices.data_ptr<int64_t>();
    a.route_weights = weights.data_ptr<float>();
    Workspace& ws = workspace_for(x, mk36_moe_workspace_bytes(&a));
    check_rc(mk36_moe_decode(&a, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return std::make_tuple(out, indices, weights);
}

// Expert-parallel partial: the rank holds experts [expert_base, expert_base + E_local) and a
// slice of the shared expert.  Returns (partial[B,H] fp32 without residual, indices, weights).
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> moe_decode_partial(
    torch::Tensor x, torch::Tensor norm_weight, torch::Tensor router_weight, torch::Tensor expert_gate, torch::Tensor expert_up,
    torch::Tensor expert_down, torch::Tensor shared_gate, torch::Tensor shared_up, torch::Tensor shared_down, double eps,
    int64_t top_k, int64_t expert_base) {
    check_moe_tensors(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down,
                      top_k, expert_gate.size(0));
    TORCH_CHECK(expert_base >= 0 && expert_base + expert_gate.size(0) <= router_weight.size(0),
                "local expert range is outside the router's experts");
    const c10::cuda::CUDAGuard guard(x.device());
    mk36_moe_args a =
        moe_args(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down, eps,
                 top_k, false);
    a.expert_base = static_cast<int32_t>(expert_base);
    a.local_experts = static_cast<int32_t>(expert_gate.size(0));
    auto partial = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kFloat32));
    auto indices = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kInt64));
    auto weights = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kFloat32));
    a.partial_out = partial.data_ptr<float>();
    a.indices = indices.data_ptr<int64_t>();
    a.route_weights = weights.data_ptr<float>();
    Workspace& ws = workspace_for(x, mk36_moe_workspace_bytes(&a));
    check_rc(mk36_moe_decode(&a, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return std::make_tuple(partial, indices, weights);
}

// Descriptor of the exchange buffers from Python integers (device pointers as mapped here).
mk36_comm comm_from(int64_t rank, int64_t world, const std::vector<int64_t>& buffers) {
    TORCH_CHECK(world >= 1 && world <= MK36_MAX_RANKS, "world size must be in [1, ", MK36_MAX_RANKS, "]");
    TORCH_CHECK(rank >= 0 && rank < world, "rank outside [0, world)");
    TORCH_CHECK(static_cast<int64_t>(buffers.size()) == world, "one exchange buffer pointer per rank is required");
    mk36_comm c{};
    c.rank = static_cast<int32_t>(rank);
    c.world = static_cast<int32_t>(world);
    for (int64_t q = 0; q < world; ++q) c.buffers[q] = reinterpret_cast<void*>(static_cast<uintptr_t>(buffers[q]));
    return c;
}

// Expert-parallel MoE step that ends, inside the kernel, with the sum over the ranks, the residual
// and the rounding: every rank returns the full output.
std::tuple<torch::Tensor, torch::Tensor, torch::Tensor> moe_decode_ep(
    torch::Tensor x, torch::Tensor norm_weight, torch::Tensor router_weight, torch::Tensor expert_gate, torch::Tensor expert_up,
    torch::Tensor expert_down, torch::Tensor shared_gate, torch::Tensor shared_up, torch::Tensor shared_down, double eps,
    int64_t top_k, bool add_residual, int64_t expert_base, int64_t rank, int64_t world, std::vector<int64_t> buffers) {
    check_moe_tensors(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down,
                      top_k, expert_gate.size(0));
    TORCH_CHECK(expert_base >= 0 && expert_base + expert_gate.size(0) <= router_weight.size(0),
                "local expert range is outside the router's experts");
    const c10::cuda::CUDAGuard guard(x.device());
    mk36_moe_args a =
        moe_args(x, norm_weight, router_weight, expert_gate, expert_up, expert_down, shared_gate, shared_up, shared_down, eps,
                 top_k, add_residual);
    a.expert_base = static_cast<int32_t>(expert_base);
    a.local_experts = static_cast<int32_t>(expert_gate.size(0));
    const mk36_comm c = comm_from(rank, world, buffers);
    auto out = torch::empty_like(x);
    auto indices = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kInt64));
    auto weights = torch::empty({x.size(0), top_k}, x.options().dtype(torch::kFloat32));
    a.out = out.data_ptr();
    a.indices = indices.data_ptr<int64_t>();
    a.route_weights = weights.data_ptr<float>();
    Workspace& ws = workspace_for(x, mk36_moe_workspace_bytes(&a));
    check_rc(mk36_moe_decode_ep(&a, &c, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return std::make_tuple(out, indices, weights);
}

int64_t comm_buffer_alloc() {
    void* p = nullptr;
    check_rc(mk36_comm_buffer_alloc(&p));
    return static_cast<int64_t>(reinterpret_cast<uintptr_t>(p));
}

void comm_buffer_reset(int64_t ptr) {
    check_rc(mk36_comm_buffer_reset(reinterpret_cast<void*>(static_cast<uintptr_t>(ptr)), at::cuda::getCurrentCUDAStream().stream()));
}

void comm_buffer_free(int64_t ptr) { check_rc(mk36_comm_buffer_free(reinterpret_cast<void*>(static_cast<uintptr_t>(ptr)))); }

py::bytes ipc_export(int64_t ptr) {
    unsigned char h[MK36_IPC_HANDLE_BYTES];
    check_rc(mk36_ipc_export(reinterpret_cast<void*>(static_cast<uintptr_t>(ptr)), h));
    return py::bytes(reinterpret_cast<const char*>(h), MK36_IPC_HANDLE_BYTES);
}

int64_t ipc_open(const std::string& handle) {
    TORCH_CHECK(handle.size() == MK36_IPC_HANDLE_BYTES, "an IPC handle has ", MK36_IPC_HANDLE_BYTES, " bytes");
    void* p = nullptr;
    check_rc(mk36_ipc_open(reinterpret_cast<const unsigned char*>(handle.data()), &p));
    return static_cast<int64_t>(reinterpret_cast<uintptr_t>(p));
}

void ipc_close(int64_t ptr) { check_rc(mk36_ipc_close(reinterpret_cast<void*>(static_cast<uintptr_t>(ptr)))); }

// -------------------------------------------------------------------------------------------
// dense_ffn_decode (no counterpart in csrc/bindings.cpp; replaces ops.py:202-218)
// -------------------------------------------------------------------------------------------
void check_dense_tensors(const torch::Tensor& x, const torch::Tensor& norm_weight, const torch::Tensor& gate_weight,
                         const torch::Tensor& up_weight, const torch::Tensor& down_weight) {
    SHIM_CHECK_INPUT(x);
    SHIM_CHECK_INPUT(norm_weight);
    SHIM_CHECK_INPUT(gate_weight);
    SHIM_CHECK_INPUT(up_weight);
    SHIM_CHECK_INPUT(down_weight);
    TORCH_CHECK(x.dim() == 2, "x must be [batch, hidden]");
    TORCH_CHECK(norm_weight.dim() == 1, "norm_weight must be [hidden]");
    TORCH_CHECK(gate_weight.dim() == 2, "gate_weight must be [intermediate, hidden]");
    TORCH_CHECK(up_weight.sizes() == gate_weight.sizes(), "up_weight shape must match gate_weight");
    TORCH_CHECK(down_weight.dim() == 2, "down_weight must be [hidden, intermediate]");
    const auto dt = x.scalar_type();
    TORCH_CHECK(dt == norm_weight.scalar_type(), "x and norm_weight dtype mismatch");
    TORCH_CHECK(dt == gate_weight.scalar_type(), "x and gate_weight dtype mismatch");
    TORCH_CHECK(dt == up_weight.scalar_type(), "x and up_weight dtype mismatch");
    TORCH_CHECK(dt == down_weight.scalar_type(), "x and down_weight dtype mismatch");
    TORCH_CHECK(norm_weight.size(0) == x.size(1), "norm_weight hidden mismatch");
    TORCH_CHECK(gate_weight.size(1) == x.size(1), "gate_weight hidden mismatch");
    TORCH_CHECK(down_weight.size(0) == x.size(1) && down_weight.size(1) == gate_weight.size(0), "down_weight shape mismatch");
}

torch::Tensor dense_ffn_impl(const torch::Tensor& x, const torch::Tensor& norm_weight, const torch::Tensor& gate_weight,
                             const torch::Tensor& up_weight, const torch::Tensor& down_weight, double eps, bool add_residual,
                             bool partial, const mk36_comm* comm = nullptr) {
    check_dense_tensors(x, norm_weight, gate_weight, up_weight, down_weight);
    const c10::cuda::CUDAGuard guard(x.device());
    mk36_dense_ffn_args a{};
    a.x = x.data_ptr();
    a.norm_weight = norm_weight.data_ptr();
    a.gate_weight = gate_weight.data_ptr();
    a.up_weight = up_weight.data_ptr();
    a.down_weight = down_weight.data_ptr();
    a.dtype = dtype_code(x, "dense_ffn_decode");
    a.batch = static_cast<int32_t>(x.size(0));
    a.hidden = static_cast<int32_t>(x.size(1));
    a.intermediate = static_cast<int32_t>(gate_weight.size(0));
    a.add_residual = add_residual ? 1 : 0;
    a.eps = static_cast<float>(eps);
    torch::Tensor out;
    if (partial) {
        out = torch::empty({x.size(0), x.size(1)}, x.options().dtype(torch::kFloat32));
        a.partial_out = out.data_ptr<float>();
    } else {
        out = torch::empty_like(x);
        a.out = out.data_ptr();
    }
    Workspace& ws = workspace_for(x, mk36_dense_ffn_workspace_bytes(&a));
    if (comm) check_rc(mk36_dense_ffn_decode_tp(&a, comm, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    else check_rc(mk36_dense_ffn_decode(&a, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

// Tensor-parallel dense FFN step (this rank's gate/up rows and down columns) that ends with the sum
// over the ranks inside the kernel.
torch::Tensor dense_ffn_decode_tp(torch::Tensor x, torch::Tensor norm_weight, torch::Tensor gate_weight, torch::Tensor up_weight,
                                  torch::Tensor down_weight, double eps, bool add_residual, int64_t rank, int64_t world,
                                  std::vector<int64_t> buffers) {
    const mk36_comm c = comm_from(rank, world, buffers);
    return dense_ffn_impl(x, norm_weight, gate_weight, up_weight, down_weight, eps, add_residual, false, &c);
}

torch::Tensor dense_ffn_decode(torch::Tensor x, torch::Tensor norm_weight, torch::Tensor gate_weight, torch::Tensor up_weight,
                               torch::Tensor down_weight, double eps, bool add_residual) {
    return dense_ffn_impl(x, norm_weight, gate_weight, up_weight, down_weight, eps, add_residual, false);
}

torch::Tensor dense_ffn_decode_partial(torch::Tensor x, torch::Tensor norm_weight, torch::Tensor gate_weight,
                                       torch::Tensor up_weight, torch::Tensor down_weight, double eps) {
    return dense_ffn_impl(x, norm_weight, gate_weight, up_weight, down_weight, eps, false, true);
}

// -------------------------------------------------------------------------------------------
// linear_decode: out = weight . (RMSNorm(x) or x) (+ residual), optionally with the arg-max of each
// output row.  Undefined tensors stand for "not given".  Returns (out, argmax or an empty tensor).
// -------------------------------------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor> linear_decode(torch::Tensor x, torch::Tensor weight, c10::optional<torch::Tensor> norm_weight,
                                                       c10::optional<torch::Tensor> residual, double eps, bool want_argmax) {
    SHIM_CHECK_INPUT(x);
    SHIM_CHECK_INPUT(weight);
    TORCH_CHECK(x.dim() == 2, "x must be [batch, in_features]");
    TORCH_CHECK(weight.dim() == 2 && weight.size(1) == x.size(1), "weight must be [out_features, in_features]");
    TORCH_CHECK(weight.scalar_type() == x.scalar_type(), "x and weight dtype mismatch");
    const c10::cuda::CUDAGuard guard(x.device());
    mk36_linear_args a{};
    a.x = x.data_ptr();
    a.weight = weight.data_ptr();
    if (norm_weight.has_value()) {
        SHIM_CHECK_INPUT(norm_weight.value());
        TORCH_CHECK(norm_weight->dim() == 1 && norm_weight->size(0) == x.size(1), "norm_weight must be [in_features]");
        TORCH_CHECK(norm_weight->scalar_type() == x.scalar_type(), "x and norm_weight dtype mismatch");
        a.norm_weight = norm_weight->data_ptr();
    }
    if (residual.has_value()) {
        SHIM_CHECK_INPUT(residual.value());
        TORCH_CHECK(residual->dim() == 2 && residual->size(0) == x.size(0) && residual->size(1) == weight.size(0),
                    "residual must be [batch, out_features]");
        TORCH_CHECK(residual->scalar_type() == x.scalar_type(), "x and residual dtype mismatch");
        a.residual = residual->data_ptr();
    }
    a.dtype = dtype_code(x, "linear_decode");
    a.batch = static_cast<int32_t>(x.size(0));
    a.in_features = static_cast<int32_t>(x.size(1));
    a.out_features = static_cast<int32_t>(weight.size(0));
    a.eps = static_cast<float>(eps);
    torch::Tensor out = torch::empty({x.size(0), weight.size(0)}, x.options());
    a.out = out.data_ptr();
    torch::Tensor best = torch::empty({want_argmax ? x.size(0) : 0}, x.options().dtype(torch::kInt64));
    if (want_argmax) a.argmax = best.data_ptr<int64_t>();
    Workspace& ws = workspace_for(x, mk36_linear_workspace_bytes(&a));
    check_rc(mk36_linear_decode(&a, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return {out, best};
}

// -------------------------------------------------------------------------------------------
// full_attention_decode: same name, arguments and return value as csrc/bindings.cpp:34.
// -------------------------------------------------------------------------------------------
torch::Tensor full_attention_decode(torch::Tensor q, torch::Tensor k_cache, torch::Tensor v_cache, double scale) {
    SHIM_CHECK_INPUT(q);
    SHIM_CHECK_INPUT(k_cache);
    SHIM_CHECK_INPUT(v_cache);
    TORCH_CHECK(q.dim() == 3, "q must be [batch, query_heads, head_dim]");
    TORCH_CHECK(k_cache.dim() == 4, "k_cache must be [batch, seq_len, kv_heads, head_dim]");
    TORCH_CHECK(v_cache.sizes() == k_cache.sizes(), "v_cache shape must match k_cache");
    TORCH_CHECK(q.scalar_type() == k_cache.scalar_type(), "q and k_cache dtype mismatch");
    TORCH_CHECK(q.scalar_type() == v_cache.scalar_type(), "q and v_cache dtype mismatch");
    TORCH_CHECK(k_cache.size(0) == q.size(0), "batch mismatch");
    TORCH_CHECK(k_cache.size(3) == q.size(2), "head_dim mismatch");
    TORCH_CHECK(q.size(1) % k_cache.size(2) == 0, "query_heads must be divisible by kv_heads");
    TORCH_CHECK(q.size(2) <= 256, "head_dim > 256 is not supported by this kernel");
    TORCH_CHECK(k_cache.size(1) > 0, "seq_len must be positive");
    const c10::cuda::CUDAGuard guard(q.device());
    mk36_attention_args a{};
    a.q = q.data_ptr();
    a.k_cache = k_cache.data_ptr();
    a.v_cache = v_cache.data_ptr();
    a.dtype = dtype_code(q, "full_attention_decode");
    a.batch = static_cast<int32_t>(q.size(0));
    a.query_heads = static_cast<int32_t>(q.size(1));
    a.kv_heads = static_cast<int32_t>(k_cache.size(2));
    a.head_dim = static_cast<int32_t>(q.size(2));
    a.seq_len = static_cast<int32_t>(k_cache.size(1));
    a.scale = static_cast<float>(scale);
    auto out = torch::empty_like(q);
    a.out = out.data_ptr();
    Workspace& ws = workspace_for(q, mk36_attention_workspace_bytes(&a));
    check_rc(mk36_full_attention_decode(&a, ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
    return out;
}

// -------------------------------------------------------------------------------------------
// linear_attention_decode: same name, arguments and return value as csrc/bindings.cpp:35.
// linear_attention_decode_ex adds per-(batch, head) decay / beta, grouped key heads and an
// optional in-place state update.
// -------------------------------------------------------------------------------------------
std::tuple<torch::Tensor, torch::Tensor> linear_attention_impl(const torch::Tensor& q, const torch::Tensor& k,
                                                               const torch::Tensor& v, const torch::Tensor& state, double decay,
                                                               const std::optional<torch::Tensor>& decay_per_head,
                                                               const std::optional<torch::Tensor>& beta_per_head, bool inplace,
                                                               bool grouped_keys) {
    SHIM_CHECK_INPUT(q);
    SHIM_CHECK_INPUT(k);
    SHIM_CHECK_INPUT(v);
    SHIM_CHECK_INPUT(state);
    TORCH_CHECK(q.dim() == 3, "q must be [batch, heads, key_dim]");
    TORCH_CHECK(k.sizes() == q.sizes(), "k shape must match q");
    TORCH_CHECK(v.dim() == 3, "v must be [batch, heads, value_dim]");
    TORCH_CHECK(state.dim() == 4, "state must be [batch, heads, key_dim, value_dim]");
    TORCH_CHECK(state.scalar_type() == torch::kFloat32, "state must be float32");
    TORCH_CHECK(q.scalar_type() == k.scalar_type(), "q and k dtype mismatch");
    TORCH_CHECK(q.scalar_type() == v.scalar_type(), "q and v dtype mismatch");
    const int64_t batch = q.size(0), key_heads = q.size(1), key_dim = q.size(2);
    const int64_t value_heads = v.size(1), value_dim = v.size(2);
    if (grouped_keys) {
        TORCH_CHECK(v.size(0) == batch && value_heads % key_heads == 0, "v batch/head mismatch");
    } else {
        TORCH_CHECK(v.size(0) == batch && value_heads == key_heads, "v batch/head mismatch");
    }
    TORCH_CHECK(state.size(0) == batch && state.size(1) == value_heads && state.size(2) == key_dim && state.size(3) == value_dim,
                "state shape mismatch");
    const c10::cuda::CUDAGuard guard(q.device());
    mk36_linear_attention_args a{};
    if (decay_per_head.has_value()) {
        const torch::Tensor& d = *decay_per_head;
        TORCH_CHECK(d.is_cuda() && d.is_contiguous() && d.scalar_type() == torch::kFloat32 && d.numel() == batch * value_heads,
                    "decay_per_head must be a contiguous float32 CUDA tensor [batch, value_heads]");
        a.decay_per_head = d.data_ptr<float>();
    }
    if (beta_per_head.has_value()) {
        const torch::Tensor& d = *beta_per_head;
        TORCH_CHECK(d.is_cuda() && d.is_contiguous() && d.scalar_type() == torch::kFloat32 && d.numel() == batch * value_heads,
                    "beta_per_head must be a contiguous float32 CUDA tensor [batch, value_heads]");
        a.beta_per_head = d.data_ptr<float>();
    }
    auto out = torch::empty({batch, value_heads, value_dim}, q.options());
    torch::Tensor new_state = inplace ? state : torch::empty_like(state);
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.state = state.data_ptr<float>();
    a.out = out.data_ptr();
    a.new_state = new_state.data_ptr<float>();
    a.dtype = dtype_code(q, "linear_attention_decode");
    a.batch = static_cast<int32_t>(batch);
    a.key_heads = static_cast<int32_t>(key_heads);
    a.value_heads = static_cast<int32_t>(value_heads);
    a.key_dim = static_cast<int32_t>(key_dim);
    a.value_dim = static_cast<int32_t>(value_dim);
    a.decay = static_cast<float>(decay);
    check_rc(mk36_linear_attention_decode(&a, at::cuda::getCurrentCUDAStream().stream()));
    return std::make_tuple(out, new_state);
}

std::tuple<torch::Tensor, torch::Tensor> linear_attention_decode(torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                                                 torch::Tensor state, double decay) {
    return linear_attention_impl(q, k, v, state, decay, std::nullopt, std::nullopt, false, false);
}

std::tuple<torch::Tensor, torch::Tensor> linear_attention_decode_ex(torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                                                    torch::Tensor state, double decay,
                                                                    std::optional<torch::Tensor> decay_per_head,
                                                                    std::optional<torch::Tensor> beta_per_head, bool inplace) {
    return linear_attention_impl(q, k, v, state, decay, decay_per_head, beta_per_head, inplace, true);
}

// Several steps in one call with the state resident on chip: q, k [steps, batch, key_heads, key_dim],
// v [steps, batch, value_heads, value_dim]; returns (out [steps, batch, value_heads, value_dim], new_state).
std::tuple<torch::Tensor, torch::Tensor> linear_attention_decode_steps(torch::Tensor q, torch::Tensor k, torch::Tensor v,
                                                                       torch::Tensor state, double decay,
                                                                       std::optional<torch::Tensor> decay_per_step,
                                                                       std::optional<torch::Tensor> beta_per_step, bool inplace) {
    SHIM_CHECK_INPUT(q);
    SHIM_CHECK_INPUT(k);
    SHIM_CHECK_INPUT(v);
    SHIM_CHECK_INPUT(state);
    TORCH_CHECK(q.dim() == 4, "q must be [steps, batch, heads, key_dim]");
    TORCH_CHECK(k.sizes() == q.sizes(), "k shape must match q");
    TORCH_CHECK(v.dim() == 4, "v must be [steps, batch, heads, value_dim]");
    TORCH_CHECK(state.dim() == 4, "state must be [batch, heads, key_dim, value_dim]");
    TORCH_CHECK(state.scalar_type() == torch::kFloat32, "state must be float32");
    TORCH_CHECK(q.scalar_type() == k.scalar_type(), "q and k dtype mismatch");
    TORCH_CHECK(q.scalar_type() == v.scalar_type(), "q and v dtype mismatch");
    const int64_t steps = q.size(0), batch = q.size(1), key_heads = q.size(2), key_dim = q.size(3);
    const int64_t value_heads = v.size(2), value_dim = v.size(3);
    TORCH_CHECK(steps > 0, "at least one step is required");
    TORCH_CHECK(v.size(0) == steps && v.size(1) == batch && value_heads % key_heads == 0, "v steps/batch/head mismatch");
    TORCH_CHECK(state.size(0) == batch && state.size(1) == value_heads && state.size(2) == key_dim && state.size(3) == value_dim,
                "state shape mismatch");
    const c10::cuda::CUDAGuard guard(q.device());
    mk36_linear_attention_steps_args a{};
    auto gate = [&](const std::optional<torch::Tensor>& g, const char* name) -> const float* {
        if (!g.has_value()) return nullptr;
        const torch::Tensor& d = *g;
        TORCH_CHECK(d.is_cuda() && d.is_contiguous() && d.scalar_type() == torch::kFloat32 && d.numel() == steps * batch * value_heads,
                    name, " must be a contiguous float32 CUDA tensor [steps, batch, value_heads]");
        return d.data_ptr<float>();
    };
    a.decay_per_step = gate(decay_per_step, "decay_per_step");
    a.beta_per_step = gate(beta_per_step, "beta_per_step");
    auto out = torch::empty({steps, batch, value_heads, value_dim}, q.options());
    torch::Tensor new_state = inplace ? state : torch::empty_like(state);
    a.q = q.data_ptr();
    a.k = k.data_ptr();
    a.v = v.data_ptr();
    a.state = state.data_ptr<float>();
    a.out = out.data_ptr();
    a.new_state = new_state.data_ptr<float>();
    a.dtype = dtype_code(q, "linear_attention_decode_steps");
    a.steps = static_cast<int32_t>(steps);
    a.batch = static_cast<int32_t>(batch);
    a.key_heads = static_cast<int32_t>(key_heads);
    a.value_heads = static_cast<int32_t>(value_heads);
    a.key_dim = static_cast<int32_t>(key_dim);
    a.value_dim = static_cast<int32_t>(value_dim);
    a.decay = static_cast<float>(decay);
    check_rc(mk36_linear_attention_decode_steps(&a, at::cuda::getCurrentCUDAStream().stream()));
    return std::make_tuple(out, new_state);
}

// Reads back the device status word of this device's workspace (synchronises the stream).
int64_t workspace_status(torch::Tensor like) {
    SHIM_CHECK_CUDA(like);
    const c10::cuda::CUDAGuard guard(like.device());
    Workspace& ws = workspace_for(like, 0);
    int status = 0;
    mk36_workspace_status(ws.buffer.data_ptr(), at::cuda::getCurrentCUDAStream().stream(), &status);
    return status;
}

void workspace_reset(torch::Tensor like) {
    SHIM_CHECK_CUDA(like);
    const c10::cuda::CUDAGuard guard(like.device());
    Workspace& ws = workspace_for(like, 0);
    check_rc(mk36_workspace_init(ws.buffer.data_ptr(), ws.bytes, at::cuda::getCurrentCUDAStream().stream()));
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
    m.def("moe_decode_persistent", &moe_decode_persistent, "Qwen3.6 persistent MoE decode kernel (sm_100a)");
    m.def("moe_decode_partial", &moe_decode_partial, "expert-parallel partial of the MoE decode kernel");
    m.def("dense_ffn_decode", &dense_ffn_decode, "Qwen3.6 dense SwiGLU FFN decode kernel (sm_100a)");
    m.def("dense_ffn_decode_partial", &dense_ffn_decode_partial, "tensor-parallel partial of the dense FFN decode kernel");
    m.def("moe_decode_ep", &moe_decode_ep, "expert-parallel MoE decode with the cross-GPU sum fused into the kernel");
    m.def("dense_ffn_decode_tp", &dense_ffn_decode_tp, "tensor-parallel dense FFN decode with the cross-GPU sum fused into the kernel");
    m.def("comm_buffer_alloc", &comm_buffer_alloc, "allocate and clear this rank's exchange buffer; returns its device pointer");
    m.def("comm_buffer_reset", &comm_buffer_reset, "clear this rank's exchange buffer on the current stream");
    m.def("comm_buffer_free", &comm_buffer_free);
    m.def("ipc_export", &ipc_export, "CUDA IPC handle of an exchange buffer");
    m.def("ipc_open", &ipc_open, "map a peer's exchange buffer; returns the device pointer in this process");
    m.def("ipc_close", &ipc_close);
    m.def("linear_decode", &linear_decode, "decode-time projection with optional fused RMSNorm, residual and arg-max (sm_100a)");
    m.def("full_attention_decode", &full_attention_decode, "Qwen3.6 full-attention decode kernel (sm_100a)");
    m.def("linear_attention_decode", &linear_attention_decode, "Qwen3.6 linear-attention recurrent decode kernel (sm_100a)");
    m.def("linear_attention_decode_ex", &linear_attention_decode_ex, "per-head decay/beta, grouped keys, optional in-place state",
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("state"), py::arg("decay") = 1.0,
          py::arg("decay_per_head") = py::none(), py::arg("beta_per_head") = py::none(), py::arg("inplace") = false);
    m.def("linear_attention_decode_steps", &linear_attention_decode_steps, "several recurrent steps in one launch, state resident on chip",
          py::arg("q"), py::arg("k"), py::arg("v"), py::arg("state"), py::arg("decay") = 1.0,
          py::arg("decay_per_step") = py::none(), py::arg("beta_per_step") = py::none(), py::arg("inplace") = false);
    m.def("workspace_status", &workspace_status, "device status word of the workspace on the tensor's device");
    m.def("workspace_reset", &workspace_reset, "re-initialise the workspace on the tensor's device");
    m.def("library_version", []() { return mk36_version(); });
}
