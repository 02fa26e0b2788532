"""Host-side behaviour that needs no GPU: configuration values, the planner, argument validation of
the operators, and that libmk36.so loads and exports every symbol include/mk36.h declares."""

import json
import re
from pathlib import Path

import pytest
import torch

import mega_kernel_qwen36 as mk
from mega_kernel_qwen36 import cabi, mpk_graph, synthetic as syn

ROOT = Path(__file__).resolve().parent.parent


# ---- configuration (values pinned by the reference's tests/test_config.py:4-41) -----------------
def test_35b_a3b_config_values():
    cfg = mk.qwen36_35b_a3b_config()
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.num_experts, cfg.num_experts_per_tok) == (2048, 40, 256, 8)
    assert (cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size) == (512, 512)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rotary_dim) == (16, 2, 256, 64)
    assert cfg.max_position_embeddings == 262144 and cfg.vocab_size == 248320
    assert (cfg.linear_num_key_heads, cfg.linear_num_value_heads) == (16, 32)
    assert (cfg.linear_key_head_dim, cfg.linear_value_head_dim, cfg.linear_conv_kernel_dim) == (128, 128, 4)
    assert cfg.layer_types[:8] == ("linear_attention",) * 3 + ("full_attention",) + ("linear_attention",) * 3 + ("full_attention",)


def test_27b_config_values():
    cfg = mk.qwen36_27b_config()
    assert cfg.model_name == "Qwen/Qwen3.6-27B" and not cfg.is_moe
    assert (cfg.hidden_size, cfg.num_hidden_layers, cfg.intermediate_size) == (5120, 64, 17408)
    assert (cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim, cfg.rotary_dim) == (24, 4, 256, 64)
    assert cfg.linear_num_value_heads == 48
    assert cfg.layer_types[3] == "full_attention" and cfg.layer_types[4] == "linear_attention"
    assert [mk.qwen36_layer_type(i) for i in range(4)] == ["linear_attention"] * 3 + ["full_attention"]


# ---- planner (behaviour pinned by the reference's tests/test_mpk_graph.py:6-49) -------------------
def test_decode_tgraph_contains_events_and_launch_modes():
    wc = mk.WorkerConfig.for_device(132)
    graph = mk.build_qwen36_decode_tgraph(mk.qwen36_27b_config(), batch_size=2, num_layers=4, worker_config=wc)
    plan = graph.linearize(worker_config=wc, batch_size=2)
    kinds = {t.kind for t in plan.graph.tasks}
    assert {"paged_attention", "linear_attention", "dense_gate_up", "dense_down", "rmsnorm"} <= kinds
    assert any(s.launch_mode == "jit" for s in plan.launch_steps)
    assert any(s.launch_mode == "aot" for s in plan.launch_steps)
    assert plan.worker_config.num_workers == 128
    assert plan.worker_config.num_local_schedulers == 16
    # every task has a trigger event whose prerequisites are its dependencies
    for t in plan.graph.tasks:
        assert plan.graph.events[t.trigger_event].prerequisites == t.depends_on
        assert t.id in plan.graph.events[t.trigger_event].dependents
    order = [s.task_id for s in plan.launch_steps]
    pos = {tid: i for i, tid in enumerate(order)}
    assert all(pos[d] < pos[t.id] for t in plan.graph.tasks for d in t.depends_on)


def test_moe_tgraph_has_router_and_grouped_experts():
    graph = mk.build_qwen36_decode_tgraph(mk.qwen36_35b_a3b_config(), batch_size=1, num_layers=1,
                                          include_sampling=False, worker_config=mk.WorkerConfig.for_device(132))
    kinds = [t.kind for t in graph.tasks]
    assert "moe_router" in kinds and "moe_grouped_experts" in kinds and "argmax" not in kinds


def test_batch_specialized_plans_use_powers_of_two():
    wc = mk.WorkerConfig.for_device(132)
    plans = mk.build_batch_specialized_plans(
        lambda b: mk.build_qwen36_decode_tgraph(mk.qwen36_27b_config(), batch_size=b, num_layers=1, worker_config=wc),
        max_batch=8, worker_config=wc)
    assert tuple(plans) == (1, 2, 4, 8)
    assert all(p.batch_size == b for b, p in plans.items())
    assert tuple(mk.build_batch_specialized_plans(lambda b: mk.build_qwen36_decode_tgraph(num_layers=1, batch_size=b),
                                                  max_batch=6)) == (1, 2, 4, 6)


def test_b200_worker_defaults_and_kernel_schedule():
    wc = mk.WorkerConfig()
    assert (wc.total_sms, wc.num_workers, wc.num_local_schedulers) == (148, 144, 16)
    cfg = mk.qwen36_35b_a3b_config()
    plan = mk.build_qwen36_decode_tgraph(cfg, batch_size=1, num_layers=4, worker_config=wc).linearize(wc, batch_size=1)
    launches = {k.name: k for k in plan.kernel_schedule}
    moe = launches["layer_0_moe"]
    assert moe.entry_point == "mk36_moe_decode" and moe.grid == 148
    assert (moe.kernel, moe.block, moe.grid_barriers, moe.launches) == ("moe_decode_stream_kernel", 416, 1, 1)
    assert moe.task_ids == ("layer_0_ffn_norm", "layer_0_moe_router_topk", "layer_0_moe_grouped_experts", "layer_0_moe_down_residual")
    assert moe.hbm_bytes == syn.moe_algorithmic_bytes(syn.MOE_35B_A3B, 1, 8) == 57_684_064
    attn = launches["layer_3_attention"]
    assert attn.entry_point == "mk36_full_attention_decode" and attn.hbm_bytes == 67_125_248
    assert launches["layer_0_linear_attention"].hbm_bytes == 4_218_880
    assert launches["layer_3_qkv_proj"].entry_point == "mk36_linear_decode"
    # every task is scheduled exactly once
    scheduled = [tid for k in plan.kernel_schedule for tid in k.task_ids]
    assert sorted(scheduled) == sorted(t.id for t in plan.graph.tasks)
    dense_plan = mk.build_qwen36_decode_tgraph(mk.qwen36_27b_config(), batch_size=8, num_layers=1).linearize(wc, batch_size=8)
    dense = {k.name: k for k in dense_plan.kernel_schedule}["layer_0_dense_ffn"]
    assert dense.hbm_bytes == syn.dense_algorithmic_bytes(syn.DENSE_27B, 8) == 534_947_840
    data = json.loads(plan.to_json())
    assert data["worker_config"]["total_sms"] == 148 and len(data["kernel_schedule"]) == len(plan.kernel_schedule)
    # the projections around the attention kernel and the LM head: launches of the projection kernel with the norms fused
    full = mk.build_qwen36_decode_tgraph(cfg, batch_size=1, num_layers=4, worker_config=wc).linearize(wc, batch_size=1)
    by_name = {k.name: k for k in full.kernel_schedule}
    qkv, outp, head = by_name["layer_3_qkv_proj"], by_name["layer_3_attn_out_proj_residual"], by_name["lm_head_argmax"]
    assert qkv.entry_point == outp.entry_point == head.entry_point == "mk36_linear_decode"
    assert qkv.task_ids == ("layer_3_attn_norm", "layer_3_qkv_proj") and head.task_ids == ("final_norm", "lm_head", "argmax_or_sampler")
    assert qkv.hbm_bytes == syn.projection_algorithmic_bytes(*syn.QKV_35B, 1, norm=True, residual=False)
    assert outp.hbm_bytes == syn.projection_algorithmic_bytes(*syn.OUT_PROJ_35B, 1, norm=False, residual=True)
    assert head.hbm_bytes == syn.projection_algorithmic_bytes(*syn.LM_HEAD_35B, 1, norm=True, residual=False)
    assert (head.kernel, head.block, head.grid_barriers, head.grid) == ("linear_decode_kernel", 288, 0, 148)
    assert by_name["layer_0_attn_norm"].entry_point is None
    # eight tokens: the batch kernel in one launch; nineteen: three launches
    plan8 = mk.build_qwen36_decode_tgraph(cfg, batch_size=8, num_layers=1, worker_config=wc).linearize(wc, batch_size=8)
    moe8 = {k.name: k for k in plan8.kernel_schedule}["layer_0_moe"]
    assert (moe8.kernel, moe8.block, moe8.grid_barriers, moe8.launches) == ("moe_decode_batch_kernel", 416, 1, 1)
    plan19 = mk.build_qwen36_decode_tgraph(cfg, batch_size=19, num_layers=1, worker_config=wc).linearize(wc, batch_size=19)
    assert {k.name: k for k in plan19.kernel_schedule}["layer_0_moe"].launches == 3
    # the ring kernel takes as many tokens per launch as its shared memory holds beside the activations
    assert mpk_graph.moe_ring_tokens_per_launch(2048, 8, 512, 512) in (1, 2, 4, 8)


def test_kernel_geometry_table_matches_the_cuda_sources():
    """The planner's launch geometry is a mirror of constants in csrc/; read them there."""
    import re

    csrc = Path(mk.__file__).resolve().parent.parent / "csrc"

    def constants(name):
        text = (csrc / name).read_text()
        found = {}
        for m in re.finditer(r"constexpr int (k\w+) = ([^;]+);", text):
            expr = m.group(2).split("//")[0].strip()
            try:
                found[m.group(1)] = int(eval(expr, {}, dict(found)))
            except Exception:
                pass
        return found

    geo = mpk_graph.KERNEL_GEOMETRY
    st = constants("mk36_moe_stream.cuh")
    assert geo["moe_decode_batch_kernel"]["block"] == st["kStThreads"]
    assert geo["moe_decode_batch_kernel"]["max_tokens"] == constants("moe_decode_batch.cu")["kBtMaxTokens"]
    assert (csrc / "moe_decode_batch.cu").read_text().count("barrier_arrive(p.ctl") == geo["moe_decode_batch_kernel"]["grid_barriers"]
    assert geo["moe_decode_stream_kernel"]["block"] == st["kStThreads"]
    assert geo["moe_decode_stream_kernel"]["max_tokens"] == 1 <= st["kStMaxTokens"]  # dispatched at one token; able to take two
    assert re.search(r"int moe_stream = 1;", (csrc / "mk36_common.cuh").read_text())
    ring = constants("moe_decode_ring.cu")
    assert geo["moe_decode_ring_kernel"]["block"] == ring["kRingThreads"]
    assert geo["moe_decode_ring_kernel"]["max_tokens"] == ring["kRingMaxTokens"]
    assert mpk_graph._RING_STAGE == ring["kRingStageBytes"]
    assert geo["dense_ffn_mma_kernel"]["block"] == constants("dense_ffn_mma.cu")["kDenseThreads"]
    assert geo["attention_decode_stream_kernel"]["block"] == constants("attention_decode_stream.cu")["kAsThreads"]
    assert geo["dense_ffn_stream_kernel"]["block"] == constants("dense_ffn_stream.cu")["kDsThreads"]
    assert geo["linear_attention_kernel"]["block"] == constants("linear_attention_decode.cu")["kLinThreads"]
    lin = constants("linear_decode.cu")
    assert geo["linear_decode_kernel"]["block"] == lin["kLinThreads"]
    assert geo["linear_decode_kernel"]["max_tokens"] == lin["kLinMaxTokens"]
    assert mpk_graph._RING_STAGE == lin["kLinStageBytes"]
    assert "barrier_arrive(" not in (csrc / "linear_decode.cu").read_text()
    # the grid barriers: one barrier_arrive per barrier in the kernel's source
    assert (csrc / "moe_decode_stream.cu").read_text().count("barrier_arrive(p.ctl") == geo["moe_decode_stream_kernel"]["grid_barriers"]
    assert (csrc / "moe_decode_ring.cu").read_text().count("barrier_arrive(p.ctl") == geo["moe_decode_ring_kernel"]["grid_barriers"]


def test_graph_rejects_duplicates_and_cycles():
    g = mk.TaskGraph(name="t")
    g.add_task("a", "linear")
    with pytest.raises(ValueError, match="duplicate task id"):
        g.add_task("a", "linear")
    g.add_task("b", "linear", depends_on=("c",))
    g.add_task("c", "linear", depends_on=("b",))
    with pytest.raises(ValueError, match="cycle or missing"):
        g.topological_tasks()


# ---- operator argument validation --------------------------------------------------------------
def _cpu_moe():
    t = syn.moe_tensors(syn.MOE_TINY, 2, seed=7, dtype=torch.float32)
    return t["x"], mk.MoeWeights(*[t[f] for f in syn.MOE_WEIGHT_FIELDS])


def test_unknown_backend_is_a_value_error():
    x, w = _cpu_moe()
    with pytest.raises(ValueError, match="backend must be one of: auto, persistent, grouped, reference"):
        mk.moe_decode(x, w, top_k=3, backend="cutlass")
    t = syn.dense_tensors(syn.DENSE_TINY, 2, seed=23, dtype=torch.float32)
    with pytest.raises(ValueError, match="backend must be one of: auto, torch, triton, reference"):
        mk.dense_ffn_decode(t["x"], mk.DenseFfnWeights(*[t[f] for f in syn.DENSE_WEIGHT_FIELDS]), backend="persistent")


def test_no_cpu_fallback():
    """CPU tensors and backend='reference' fail loudly; nothing is computed by PyTorch."""
    x, w = _cpu_moe()
    for backend in ("auto", "persistent", "grouped"):
        with pytest.raises(RuntimeError, match="no CPU path|not built"):
            mk.moe_decode(x, w, top_k=3, backend=backend)
    with pytest.raises(RuntimeError, match="not part of this package"):
        mk.moe_decode(x, w, top_k=3, backend="reference")
    q = torch.zeros(1, 2, 8)
    with pytest.raises(RuntimeError, match="no CPU path|not built"):
        mk.full_attention_decode(mk.FullAttentionInputs(q=q, k_cache=torch.zeros(1, 3, 1, 8), v_cache=torch.zeros(1, 3, 1, 8)))
    with pytest.raises(RuntimeError, match="no CPU path|not built"):
        mk.linear_attention_decode(mk.LinearAttentionInputs(q=q, k=q, v=q, state=torch.zeros(1, 2, 8, 8)))
    with pytest.raises(ValueError, match="unsupported layer_type"):
        mk.decode_layer(0, x, w, layer_type="sliding_window")


def test_dataclass_field_order_matches_the_native_argument_order():
    assert [f for f in mk.MoeWeights.__dataclass_fields__] == list(syn.MOE_WEIGHT_FIELDS)
    assert [f for f in mk.DenseFfnWeights.__dataclass_fields__] == list(syn.DENSE_WEIGHT_FIELDS)
    fa = mk.FullAttentionInputs(q=None, k_cache=None, v_cache=None)
    assert (fa.cos, fa.sin, fa.rotary_dim, fa.scale) == (None, None, 64, None)
    assert mk.LinearAttentionInputs(q=None, k=None, v=None, state=None).decay == 1.0


# ---- C ABI ------------------------------------------------------------------------------------
def _declared_symbols():
    text = (ROOT / "include" / "mk36.h").read_text()
    return sorted(set(re.findall(r"MK36_API\s+[\w\s\*]+?\b(mk36_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    declared = _declared_symbols()
    assert len(declared) >= 13
    assert sorted(cabi.SIGNATURES) == declared, "cabi.SIGNATURES and include/mk36.h disagree"
    lib = cabi.load()
    for name in declared:
        assert hasattr(lib, name), f"libmk36.so does not export {name}"
    assert lib.mk36_version() >= 100
    assert lib.mk36_workspace_bytes() >= 1 << 20


def test_extension_module_exposes_the_reference_entry_points():
    assert mk.extension_available()
    from mega_kernel_qwen36 import _C

    for name in ("moe_decode_persistent", "full_attention_decode", "linear_attention_decode", "dense_ffn_decode"):
        assert hasattr(_C, name)


def test_c_abi_argument_errors_need_no_gpu():
    lib = cabi.load()
    assert lib.mk36_moe_decode(None, None, 0, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"args is NULL" in lib.mk36_last_error()
    args = cabi.AttentionArgs(q=1, k_cache=1, v_cache=1, out=1, dtype=cabi.MK36_BF16, batch=1, query_heads=3, kv_heads=2,
                              head_dim=64, seq_len=5, scale=1.0)
    assert lib.mk36_full_attention_decode(args, None, 0, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"divisible by kv_heads" in lib.mk36_last_error()
    args.query_heads, args.head_dim = 4, 512
    assert lib.mk36_full_attention_decode(args, None, 0, None) == cabi.MK36_ERR_UNSUPPORTED
    la = cabi.LinearAttentionArgs(q=1, k=1, v=1, state=1, out=1, new_state=1, dtype=0, batch=1, key_heads=3, value_heads=4,
                                  key_dim=8, value_dim=8, decay=1.0)
    assert lib.mk36_linear_attention_decode(la, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"multiple of key_heads" in lib.mk36_last_error()
    assert lib.mk36_workspace_init(None, 0, None) == cabi.MK36_ERR_WORKSPACE
    # multi-step recurrence and the multi-GPU entry points refuse bad descriptors before touching a device
    ls = cabi.LinearAttentionStepsArgs(q=1, k=1, v=1, state=1, out=1, new_state=1, dtype=0, steps=0, batch=1, key_heads=2,
                                       value_heads=4, key_dim=8, value_dim=8, decay=1.0)
    assert lib.mk36_linear_attention_decode_steps(ls, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"sizes must be positive" in lib.mk36_last_error()
    ls.steps, ls.key_heads = 4, 3
    assert lib.mk36_linear_attention_decode_steps(ls, None) == cabi.MK36_ERR_INVALID_ARG
    assert lib.mk36_moe_decode_ep(None, None, None, 0, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"comm is NULL" in lib.mk36_last_error()
    assert lib.mk36_dense_ffn_decode_tp(None, None, None, 0, None) == cabi.MK36_ERR_INVALID_ARG
    assert lib.mk36_ipc_export(None, None) == cabi.MK36_ERR_INVALID_ARG
    assert lib.mk36_ipc_open(None, None) == cabi.MK36_ERR_INVALID_ARG
    assert lib.mk36_comm_buffer_alloc(None) == cabi.MK36_ERR_INVALID_ARG
    assert lib.mk36_comm_buffer_bytes() >= 2 * 8 * 8 * 8192 * 8
    assert lib.mk36_full_attention_decode_static(None, None) == cabi.MK36_ERR_INVALID_ARG


def test_algorithmic_byte_formulas():
    assert syn.moe_algorithmic_bytes(syn.MOE_35B_A3B, 8, 64) == 410_063_616
    assert syn.dense_algorithmic_bytes(syn.DENSE_27B, 1) == 534_804_480
    assert syn.attention_algorithmic_bytes(1, 16, 2, 256, 32768) == 67_125_248
    assert syn.attention_algorithmic_bytes(1, 16, 2, 256, 4096) == 8_404_992
    assert syn.linear_algorithmic_bytes(8, 16, 32, 128, 128) == 33_751_040


def test_ctypes_structures_match_the_c_header(tmp_path):
    """Size and field offsets of every argument struct, as the C compiler sees include/mk36.h,
    against the ctypes mirror in cabi.py (a drifted field would otherwise only show on a GPU)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc") or shutil.which("cc")
    if gcc is None:
        pytest.skip("no C compiler")
    pairs = {
        "mk36_moe_args": cabi.MoeArgs,
        "mk36_dense_ffn_args": cabi.DenseFfnArgs,
        "mk36_attention_args": cabi.AttentionArgs,
        "mk36_linear_attention_args": cabi.LinearAttentionArgs,
        "mk36_linear_attention_steps_args": cabi.LinearAttentionStepsArgs,
        "mk36_comm": cabi.Comm,
    }
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "mk36.h"', "int main(void) {"]
    for cname, ctype in pairs.items():
        lines.append(f'printf("{cname} size %zu\\n", sizeof({cname}));')
        for field, _ in ctype._fields_:
            lines.append(f'printf("{cname} {field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["return 0; }"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines))
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-I", str(ROOT / "include"), str(src), "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], check=True, capture_output=True, text=True).stdout
    seen = {}
    for line in out.splitlines():
        cname, field, value = line.split()
        seen[(cname, field)] = int(value)
    for cname, ctype in pairs.items():
        assert seen[(cname, "size")] == __import__("ctypes").sizeof(ctype), cname
        for field, _ in ctype._fields_:
            assert seen[(cname, field)] == getattr(ctype, field).offset, f"{cname}.{field}"


def test_extension_errors_with_formatted_numbers_raise_instead_of_crashing():
    """An error message that formats a number goes through the C++ stream machinery of the extension;
    an extension linked against a private static copy of the C++ runtime crashed there.  Run in a child
    process so that a crash is a failure of this test only."""
    import subprocess
    import sys

    if not mk.extension_available():
        pytest.skip("extension not built")
    code = (
        "import sys; sys.path.insert(0, %r)\n"
        "import torch\n"
        "from mega_kernel_qwen36 import _C as ext\n"
        "try:\n"
        "    ext.ipc_open('abc')\n"
        "except RuntimeError as e:\n"
        "    assert '64 bytes' in str(e), str(e)\n"
        "    print('raised')\n"
    ) % str(Path(mk.__file__).resolve().parent.parent)
    proc = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert proc.returncode == 0 and "raised" in proc.stdout, (proc.returncode, proc.stderr[-500:])


def test_exchange_buffer_reset_checks_its_argument():
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    assert lib.mk36_comm_buffer_reset(None, None) == cabi.MK36_ERR_INVALID_ARG
    assert b"buffer is NULL" in lib.mk36_last_error()
