"""CUDA kernels against the CPU oracle and the reference fixtures, on identical seeded inputs.

Every call goes through the public operators, i.e. through the extension shim and the C ABI of
libmk36.so.  Tolerances (tests/parity.py): outputs max-abs <= 2e-2 (or one unit in the last
place of the output dtype where that is larger) and rel-L2 <= 1e-2; top-k indices bit-exact;
fp32 recurrent state <= 1e-4 relative after each of 64 steps.
"""

import numpy as np
import pytest
import torch

from golden_cases import CASES, CASES_BY_NAME
from parity import assert_indices_exact, assert_output_parity, assert_state_parity, rel_l2
from runners import assert_same_inputs, build_inputs, golden_state_sample, load_golden, run_cuda, run_oracle
from test_golden import check_oracle_against_fixture

pytestmark = pytest.mark.gpu

FAST = [c for c in CASES if c.op != "linear"]
LINEAR = [c for c in CASES if c.op == "linear"]


def _margin(case, spec):
    from oracle import decode_oracle as oracle
    from mega_kernel_qwen36 import synthetic as syn

    t = spec["tensors"]
    _, _, _, logits = oracle.moe_decode_f64(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=spec["top_k"])
    return oracle.router_margin(logits, spec["top_k"])


@pytest.mark.parametrize("case", FAST, ids=lambda c: c.name)
def test_kernel_matches_oracle_and_fixture(case, cuda_device):
    spec = build_inputs(case)
    golden = load_golden(case.name)
    assert_same_inputs(case, spec, golden)
    got = run_cuda(case, spec, cuda_device)
    ref = run_oracle(case, spec)
    # the oracle on this host against the stored output of the reference's own reference.py
    check_oracle_against_fixture(case, ref, golden)
    if case.op == "moe":
        if not torch.equal(got["indices"], ref["indices"]):
            assert_indices_exact(got["indices"], ref["indices"], margin=_margin(case, spec))
        assert got["indices"].dtype == torch.int64
        torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
        torch.testing.assert_close(got["weights"].sum(-1), torch.ones(got["weights"].shape[0]), atol=1e-5, rtol=0)
    assert got["out"].dtype == ref["out"].dtype
    assert_output_parity(got["out"], ref["out"], what=case.name)
    assert_output_parity(got["out"], torch.from_numpy(golden["out"]).to(got["out"].dtype), what=case.name + " vs fixture")


GENERIC_PATH_CASES = ["moe_small_bf16_b3", "moe_small_f16_b2", "moe_tiny_bf16_b11", "moe_35b_bf16_b1_s0", "moe_35b_bf16_b8_s0"]


@pytest.mark.parametrize("name", GENERIC_PATH_CASES)
def test_moe_general_kernel_matches_oracle(name, cuda_device):
    """Shapes that normally take the shared-memory-ring variant, forced through the general
    register-streaming kernel: both must meet the same tolerances."""
    from mega_kernel_qwen36 import cabi

    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    lib = cabi.load()
    cabi.check(lib.mk36_set_option(b"force_generic", 1))
    try:
        got = run_cuda(case, spec, cuda_device)
    finally:
        cabi.check(lib.mk36_set_option(b"force_generic", 0))
    ref = run_oracle(case, spec)
    assert_indices_exact(got["indices"], ref["indices"])
    torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
    assert_output_parity(got["out"], ref["out"], what=name + " (general kernel)")
    assert lib.mk36_set_option(b"no_such_option", 1) == cabi.MK36_ERR_INVALID_ARG


@pytest.mark.parametrize("name", ["moe_small_bf16_b3", "moe_small_f16_b2", "moe_35b_bf16_b1_s0", "moe_35b_bf16_b8_s1"])
def test_moe_ring_kernel_tensor_core_consumers_match_oracle(name, cuda_device):
    """The ring kernel contracts with plain FMAs for launches of up to four tokens and with
    mma.sync beyond; the switch forces the tensor-core consumers on the small launches as well."""
    from mega_kernel_qwen36 import cabi

    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    lib = cabi.load()
    cabi.check(lib.mk36_set_option(b"ring_mma", 1))
    try:
        got = run_cuda(case, spec, cuda_device)
    finally:
        cabi.check(lib.mk36_set_option(b"ring_mma", 0))
    ref = run_oracle(case, spec)
    assert_indices_exact(got["indices"], ref["indices"])
    torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
    assert_output_parity(got["out"], ref["out"], what=name + " (tensor-core consumers)")


MOE_DEFAULT_OPTIONS = {"moe_stream": 1, "moe_batch": 1, "moe_static": 0, "moe_stages": 0, "moe_dyn_rounds": 0}


def _run_with_options(case, spec, device, options):
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    pairs = [o.split("=") for o in options.split(",")]
    for key, value in pairs:
        cabi.check(lib.mk36_set_option(key.encode(), int(value)))
    try:
        return run_cuda(case, spec, device)
    finally:
        for key, _ in pairs:
            cabi.check(lib.mk36_set_option(key.encode(), MOE_DEFAULT_OPTIONS[key]))


@pytest.mark.parametrize("name", ["moe_small_f16_b2", "moe_35b_bf16_b1_s0", "moe_35b_bf16_b2_s0"])
@pytest.mark.parametrize("option", ["moe_stream=2", "moe_stream=0", "moe_stream=0,moe_batch=0", "moe_stream=2,moe_static=1",
                                    "moe_stream=2,moe_stages=3", "moe_stream=2,moe_dyn_rounds=7"])
def test_moe_small_batch_kernel_variants_match_oracle(name, option, cuda_device):
    """One-token calls run the stream kernel and two-token calls the batch kernel; the same calls through the
    stream kernel at two tokens, the batch kernel at one, the ring kernel's plain-FMA consumers, and the stream
    kernel with statically dealt chunks, a shallower ring or all rounds dealt through the counter must meet
    the same tolerances."""
    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    got = _run_with_options(case, spec, cuda_device, option)
    ref = run_oracle(case, spec)
    assert_indices_exact(got["indices"], ref["indices"])
    torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
    assert_output_parity(got["out"], ref["out"], what=f"{name} ({option})")


@pytest.mark.parametrize("name", ["moe_small_bf16_b3", "moe_35b_bf16_b4_s0", "moe_35b_bf16_b8_s2"])
@pytest.mark.parametrize("option", ["moe_batch=0", "moe_static=1", "moe_stages=3", "moe_dyn_rounds=6"])
def test_moe_batch_kernel_variants_match_oracle(name, option, cuda_device):
    """Calls of two or more tokens run the batch kernel (eight tokens per launch); the same calls
    through the ring kernel, and the batch kernel with statically dealt chunks, a shallower ring or more
    rounds dealt through the counter, must meet the same tolerances."""
    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    got = _run_with_options(case, spec, cuda_device, option)
    ref = run_oracle(case, spec)
    assert_indices_exact(got["indices"], ref["indices"])
    torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
    assert_output_parity(got["out"], ref["out"], what=f"{name} ({option})")


@pytest.mark.parametrize("shape,batch,dtype,same", [
    ("small", 5, torch.float16, False),
    ("small", 8, torch.bfloat16, True),
    ("35b", 3, torch.bfloat16, False),
    ("35b", 7, torch.bfloat16, False),
    ("35b", 8, torch.bfloat16, True),
    ("35b", 9, torch.bfloat16, False),
    ("35b", 19, torch.bfloat16, False),
], ids=lambda v: str(v).replace("torch.", ""))
def test_moe_batch_kernel_ragged_and_shared_experts(shape, batch, dtype, same, cuda_device):
    """Token counts that do not fill a launch of eight (3, 5, 7), that need a second and third launch
    with a remainder (9 = 8 + 1, 19 = 8 + 8 + 3), and eight identical tokens, which all choose the
    same experts, so that every expert block meets all eight activation vectors."""
    from golden_cases import Case
    from mega_kernel_qwen36 import synthetic as syn

    shp = syn.MOE_SMALL if shape == "small" else syn.MOE_35B_A3B
    t = syn.moe_tensors(shp, batch, 11 + batch, dtype)
    if same:
        t["x"] = t["x"][:1].repeat(batch, 1).contiguous()
    case = Case(f"moe_{shape}_b{batch}", "moe", lambda: None)
    spec = {"tensors": t, "top_k": shp.top_k}
    got = run_cuda(case, spec, cuda_device)
    ref = run_oracle(case, spec)
    assert_indices_exact(got["indices"], ref["indices"])
    torch.testing.assert_close(got["weights"], ref["weights"], atol=1e-5, rtol=1e-4)
    assert_output_parity(got["out"], ref["out"], what=case.name)
    if same:
        assert torch.equal(got["out"], got["out"][:1].expand_as(got["out"])), "identical tokens must give identical rows"


@pytest.mark.parametrize("batch", [1, 2, 8])
def test_moe_equal_logits_go_to_the_lowest_expert_index(batch, cuda_device):
    """Router rows e and e + 128 are made identical, and so are rows 5 and 70, so that every logit has a
    bit-equal twin: in the same lane of the selecting warp (e and e + 128) and in another lane (5 and 70).
    Selection order: descending logit, lowest expert index among equals; the eight winners are then four
    pairs of twins, each pair in index order."""
    from golden_cases import Case
    from oracle import decode_oracle as oracle
    from mega_kernel_qwen36 import synthetic as syn

    shp = syn.MOE_35B_A3B
    t = syn.moe_tensors(shp, batch, 5, torch.bfloat16)
    rw = t["router_weight"].clone()
    rw[128:] = rw[:128]
    rw[70] = rw[5]
    rw[198] = rw[5]
    t["router_weight"] = rw
    spec = {"tensors": t, "top_k": shp.top_k}
    got = run_cuda(Case("moe_ties", "moe", lambda: None), spec, cuda_device)
    _, _, _, logits = oracle.moe_decode_f64(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=shp.top_k)
    order = torch.sort(logits, dim=-1, descending=True, stable=True).indices[:, : shp.top_k]
    # the margin between the eighth and the ninth *distinct* logit decides whether fp32 and fp64 can disagree
    for b in range(batch):
        distinct = torch.sort(torch.unique(logits[b]), descending=True).values
        assert float((distinct[:5] - distinct[1:6]).min()) > 1e-5
    assert torch.equal(got["indices"], order), (got["indices"], order)
    ref = oracle.moe_decode_f64(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=shp.top_k, indices=order)[0]
    assert_output_parity(got["out"], ref.to(got["out"].dtype), what="moe with tied logits")


@pytest.mark.parametrize("name", ["dense_mid_f16_b1", "dense_27b_bf16_b1"])
def test_dense_one_token_through_the_tensor_core_kernel(name, cuda_device):
    """One-token dense FFN calls run the streaming kernel; the tensor-core kernel that serves larger
    batches must give the same call the same answer within the tolerances."""
    from mega_kernel_qwen36 import cabi

    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    lib = cabi.load()
    cabi.check(lib.mk36_set_option(b"dense_stream", 0))
    try:
        got = run_cuda(case, spec, cuda_device)
    finally:
        cabi.check(lib.mk36_set_option(b"dense_stream", 1))
    assert_output_parity(got["out"], run_oracle(case, spec)["out"], what=name + " (tensor-core kernel)")


@pytest.mark.parametrize("name", ["attn_27b_bf16_t1000", "attn_35b_bf16_t4096", "attn_35b_bf16_b2_t2500"])
def test_attention_general_kernel_matches_oracle(name, cuda_device):
    """Shapes that normally take the tensor-core attention kernel, forced through the general one."""
    from mega_kernel_qwen36 import cabi

    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    lib = cabi.load()
    cabi.check(lib.mk36_set_option(b"force_generic", 1))
    try:
        got = run_cuda(case, spec, cuda_device)
    finally:
        cabi.check(lib.mk36_set_option(b"force_generic", 0))
    assert_output_parity(got["out"], run_oracle(case, spec)["out"], what=name + " (general kernel)")


@pytest.mark.parametrize("name", ["attn_tiny_bf16_t128", "attn_27b_bf16_t1000", "attn_35b_bf16_t4096", "attn_35b_bf16_b2_t2500"])
def test_attention_register_staged_kernel_matches_oracle(name, cuda_device):
    """Shapes that normally take the streaming attention kernel (shared-memory ring), forced through the
    tensor-core kernel that stages the cache in registers: same tolerances."""
    from mega_kernel_qwen36 import cabi

    case = CASES_BY_NAME[name]
    spec = build_inputs(case)
    lib = cabi.load()
    cabi.check(lib.mk36_set_option(b"attn_stream", 0))
    try:
        got = run_cuda(case, spec, cuda_device)
    finally:
        cabi.check(lib.mk36_set_option(b"attn_stream", 1))
    assert_output_parity(got["out"], run_oracle(case, spec)["out"], what=name + " (register-staged kernel)")


@pytest.mark.parametrize("seq", [1, 2, 3, 17])
def test_attention_short_context_keeps_its_weights_normalised(seq, cuda_device):
    """A few cached tokens: nothing averages out, so the soft-max weights must add up to one exactly as
    they are applied (the kernel rounds them to bf16 for the tensor-core product and sums the
    normaliser from the rounded values).  Held to a tighter relative-L2 bound than the general one:
    4e-3, where the rounding of the bf16 output alone is about 2e-3."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    t = syn.attention_tensors(2, 16, 2, 256, seq, seed=40 + seq)
    ref = oracle.full_attention_decode(t["q"], t["k_cache"], t["v_cache"], scale=1.0 / 16)
    got = mk.full_attention_decode(mk.FullAttentionInputs(q=t["q"].to(cuda_device), k_cache=t["k_cache"].to(cuda_device),
                                                          v_cache=t["v_cache"].to(cuda_device), scale=1.0 / 16)).cpu()
    assert_output_parity(got, ref, what=f"attention T={seq}", rel_l2_tol=4e-3)


@pytest.mark.parametrize("case", LINEAR, ids=lambda c: c.name)
def test_linear_attention_state_drift(case, cuda_device):
    """64 consecutive steps, feeding the new state back: state error after every step, outputs at
    every step, and the fixture's final-state sample."""
    import mega_kernel_qwen36 as mk
    from oracle import decode_oracle as oracle

    spec = build_inputs(case)
    golden = load_golden(case.name)
    assert_same_inputs(case, spec, golden)
    s_ref = spec["state"]
    s_gpu = spec["state"].to(cuda_device)
    s_in_copy = s_gpu.clone()
    worst = 0.0
    for si, step in enumerate(spec["steps"]):
        q = step["q"].repeat_interleave(spec["expand"], dim=1)
        k = step["k"].repeat_interleave(spec["expand"], dim=1)
        o_ref, s_ref = oracle.linear_attention_decode(q, k, step["v"], s_ref, decay=spec["decay"])
        prev = s_gpu
        o_gpu, s_gpu = mk.linear_attention_decode(mk.LinearAttentionInputs(
            q=q.to(cuda_device), k=k.to(cuda_device), v=step["v"].to(cuda_device), state=s_gpu, decay=spec["decay"]))
        if si == 0:
            assert torch.equal(prev, s_in_copy), "the input state must not be modified"
            assert s_gpu.data_ptr() != prev.data_ptr()
        worst = max(worst, assert_state_parity(s_gpu, s_ref, what=f"{case.name} step {si}"))
        assert_output_parity(o_gpu.cpu(), o_ref, what=f"{case.name} out step {si}")
    assert s_gpu.dtype == torch.float32
    # the multiply / add are rounded separately as in the reference, so the state is bit-exact
    assert torch.equal(s_gpu.cpu(), s_ref), f"state not bit-exact (rel {worst:.3g})"
    np.testing.assert_array_equal(golden_state_sample(s_gpu), golden["state_sample"])


def test_linear_attention_per_head_gates_and_grouped_keys(cuda_device):
    """16 key heads serving 32 value heads, per-(batch, head) decay g and value scale beta, over 64
    consecutive steps with the state fed back (the state drift bound holds after every step)."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    B, HK, HV, DK, DV = 2, 16, 32, 128, 128
    s_ref = syn.linear_state(B, HV, DK, DV, seed=5)
    s_gpu = s_ref.to(cuda_device)
    for si, step in enumerate(syn.linear_step_stream(B, HK, HV, DK, DV, steps=64, seed=5)):
        o_ref, s_ref = oracle.linear_attention_decode_per_head(step["q"], step["k"], step["v"], s_ref, step["g"], step["beta"])
        o_gpu, s_gpu = mk.linear_attention_decode_gated(
            step["q"].to(cuda_device), step["k"].to(cuda_device), step["v"].to(cuda_device), s_gpu,
            decay_per_head=step["g"].to(cuda_device), beta_per_head=step["beta"].to(cuda_device), inplace=(si % 2 == 1))
        assert_state_parity(s_gpu, s_ref, what=f"gated step {si}")
        assert_output_parity(o_gpu.cpu(), o_ref, what=f"gated out step {si}")


@pytest.mark.parametrize("case", LINEAR, ids=lambda c: c.name)
def test_linear_attention_multi_step_matches_step_by_step(case, cuda_device):
    """All 64 steps in one launch (state resident on chip): outputs and final state bit-identical to
    the step-by-step kernel, hence the same parity with the oracle and the fixture."""
    import mega_kernel_qwen36 as mk
    from oracle import decode_oracle as oracle

    spec = build_inputs(case)
    golden = load_golden(case.name)
    qs = torch.stack([s["q"] for s in spec["steps"]]).to(cuda_device)
    ks = torch.stack([s["k"] for s in spec["steps"]]).to(cuda_device)
    vs = torch.stack([s["v"] for s in spec["steps"]]).to(cuda_device)
    state0 = spec["state"].to(cuda_device)
    keep = state0.clone()
    # key heads are given as they are (fewer than value heads where the case says so)
    outs, final = mk.linear_attention_decode_steps(qs, ks, vs, state0, decay=spec["decay"])
    assert torch.equal(state0, keep), "the input state must not be modified"
    s_ref = spec["state"]
    s_gpu = state0
    for si, step in enumerate(spec["steps"]):
        q = step["q"].repeat_interleave(spec["expand"], dim=1)
        k = step["k"].repeat_interleave(spec["expand"], dim=1)
        o_ref, s_ref = oracle.linear_attention_decode(q, k, step["v"], s_ref, decay=spec["decay"])
        o_one, s_gpu = mk.linear_attention_decode(mk.LinearAttentionInputs(
            q=q.to(cuda_device), k=k.to(cuda_device), v=step["v"].to(cuda_device), state=s_gpu, decay=spec["decay"]))
        assert torch.equal(outs[si], o_one), f"{case.name}: step {si} differs from the single-step kernel"
        assert_output_parity(outs[si].cpu(), o_ref, what=f"{case.name} multi-step out {si}")
    assert torch.equal(final, s_gpu)
    assert torch.equal(final.cpu(), s_ref)
    np.testing.assert_array_equal(golden_state_sample(final), golden["state_sample"])


def test_linear_attention_multi_step_gates_in_place(cuda_device):
    """Per-step, per-head decay and beta, grouped key heads, in-place state."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    B, HK, HV, DK, DV, T = 2, 16, 32, 128, 128, 64
    steps = list(syn.linear_step_stream(B, HK, HV, DK, DV, steps=T, seed=6))
    s_ref = syn.linear_state(B, HV, DK, DV, seed=6)
    state = s_ref.to(cuda_device)
    stack = lambda name: torch.stack([s[name] for s in steps]).to(cuda_device)
    outs, final = mk.linear_attention_decode_steps(stack("q"), stack("k"), stack("v"), state, decay_per_step=stack("g"),
                                                   beta_per_step=stack("beta"), inplace=True)
    assert final.data_ptr() == state.data_ptr()
    for si, step in enumerate(steps):
        o_ref, s_ref = oracle.linear_attention_decode_per_head(step["q"], step["k"], step["v"], s_ref, step["g"], step["beta"])
        assert_output_parity(outs[si].cpu(), o_ref, what=f"multi-step gated out {si}")
    assert_state_parity(final, s_ref, what="multi-step gated final state")
    # shapes off the fast path (value_dim not a multiple of 4) take the step-by-step route inside the library
    tiny = list(syn.linear_step_stream(2, 3, 3, 5, 7, steps=3, seed=2, dtype=torch.float32))
    s_ref = syn.linear_state(2, 3, 5, 7, seed=2)
    tq, tk, tv = (torch.stack([s[n] for s in tiny]).to(cuda_device) for n in ("q", "k", "v"))
    outs, final = mk.linear_attention_decode_steps(tq, tk, tv, s_ref.to(cuda_device), decay=0.9)
    for si, step in enumerate(tiny):
        o_ref, s_ref = oracle.linear_attention_decode(step["q"], step["k"], step["v"], s_ref, decay=0.9)
        assert_output_parity(outs[si].cpu(), o_ref, what=f"multi-step tiny out {si}")
    assert_state_parity(final, s_ref, what="multi-step tiny final state")


def test_moe_runs_are_bit_identical(cuda_device):
    """All reductions have a fixed order: 20 runs give the same bits (a race would not)."""
    case = CASES_BY_NAME["moe_small_bf16_b3"]
    spec = build_inputs(case)
    first = run_cuda(case, spec, cuda_device)
    for _ in range(19):
        again = run_cuda(case, spec, cuda_device)
        assert torch.equal(first["out"], again["out"])
        assert torch.equal(first["indices"], again["indices"])
        assert torch.equal(first["weights"], again["weights"])


def test_attention_runs_are_bit_identical(cuda_device):
    case = CASES_BY_NAME["attn_odd_bf16_t777"]
    spec = build_inputs(case)
    first = run_cuda(case, spec, cuda_device)
    for _ in range(9):
        assert torch.equal(first["out"], run_cuda(case, spec, cuda_device)["out"])


def test_moe_without_residual_and_repeated_rows(cuda_device):
    """add_residual=False, and a batch whose rows are all equal (every token picks the same experts,
    so one distinct expert serves 8 tokens)."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    t = syn.moe_tensors(syn.MOE_SMALL, 1, seed=3, dtype=torch.bfloat16)
    t["x"] = t["x"].repeat(8, 1).contiguous()
    ref, ridx, rw = oracle.moe_decode(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=4, add_residual=False)
    d = {k: v.to(cuda_device) for k, v in t.items()}
    out, idx, w = mk.moe_decode(d["x"], mk.MoeWeights(*[d[f] for f in syn.MOE_WEIGHT_FIELDS]), top_k=4, add_residual=False)
    assert_indices_exact(idx, ridx)
    assert_output_parity(out.cpu(), ref, what="moe no-residual")


def test_decode_layer_wiring(cuda_device):
    """decode_layer = token mixer + residual + FFN with residual, for both layer kinds and both FFNs."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    B, H = 2, 256
    moe_t = syn.moe_tensors(syn.MOE_SMALL, B, seed=21)
    dense_t = syn.dense_tensors(syn.DenseShape(256, 704), B, seed=22)
    hidden = moe_t["x"]
    attn = syn.attention_tensors(B, 8, 2, 32, 300, seed=23)          # 8 heads x 32 = 256 = hidden
    lin = {"q": None}
    step = next(syn.linear_step_stream(B, 4, 4, 64, 64, steps=1, seed=24))  # 4 heads x 64 = 256
    state = syn.linear_state(B, 4, 64, 64, seed=24)
    dev = cuda_device
    moe_w = mk.MoeWeights(*[moe_t[f].to(dev) for f in syn.MOE_WEIGHT_FIELDS])
    dense_w = mk.DenseFfnWeights(*[dense_t[f].to(dev) for f in syn.DENSE_WEIGHT_FIELDS])

    # layer 3: full attention + MoE
    r = mk.decode_layer(3, hidden.to(dev), moe_w, top_k=4,
                        full_attention=mk.FullAttentionInputs(q=attn["q"].to(dev), k_cache=attn["k_cache"].to(dev),
                                                              v_cache=attn["v_cache"].to(dev)))
    o = oracle.decode_layer(3, hidden, moe=[moe_t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=4,
                            full_attention={"q": attn["q"], "k_cache": attn["k_cache"], "v_cache": attn["v_cache"]})
    assert r.linear_state is None and r.attention_output is not None
    assert_indices_exact(r.router_indices, o["router_indices"])
    assert_output_parity(r.hidden.cpu(), o["hidden"], what="layer 3 hidden")

    # layer 0: linear attention + dense FFN
    r = mk.decode_layer(0, hidden.to(dev), dense_ffn=dense_w,
                        linear_attention=mk.LinearAttentionInputs(q=step["q"].to(dev), k=step["k"].to(dev),
                                                                  v=step["v"].to(dev), state=state.to(dev), decay=0.95))
    o = oracle.decode_layer(0, hidden, dense=[dense_t[f] for f in syn.DENSE_WEIGHT_FIELDS],
                            linear_attention={"q": step["q"], "k": step["k"], "v": step["v"], "state": state, "decay": 0.95})
    assert r.router_indices is None and r.linear_state is not None
    assert_state_parity(r.linear_state, o["linear_state"])
    assert_output_parity(r.hidden.cpu(), o["hidden"], what="layer 0 hidden")

    with pytest.raises(ValueError, match="full_attention inputs are required"):
        mk.decode_layer(3, hidden.to(dev), moe_w)
    with pytest.raises(ValueError, match="either moe or dense_ffn weights are required"):
        mk.decode_layer(0, hidden.to(dev), linear_attention=mk.LinearAttentionInputs(
            q=step["q"].to(dev), k=step["k"].to(dev), v=step["v"].to(dev), state=state.to(dev)))
    del lin


def test_attention_with_partial_rope(cuda_device):
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    t = syn.attention_tensors(1, 4, 2, 64, 50, seed=31)
    ang = torch.linspace(0, 3, 16).repeat(2)
    cos, sin = torch.cos(ang), torch.sin(ang)
    q2, k2 = oracle.apply_partial_rope(t["q"], t["k_cache"], cos, sin, 32)
    ref = oracle.full_attention_decode(q2, k2, t["v_cache"])
    dev = cuda_device
    got = mk.full_attention_decode(mk.FullAttentionInputs(q=t["q"].to(dev), k_cache=t["k_cache"].to(dev),
                                                          v_cache=t["v_cache"].to(dev), cos=cos, sin=sin, rotary_dim=32))
    assert_output_parity(got.cpu(), ref, what="attention with rope")


def test_error_behaviour_on_device(cuda_device):
    """Same exception types and message fragments as the reference's checks
    (csrc/persistent_moe_decode.cu:668-696, tests/test_cuda_ops.py:52-65)."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    dev = cuda_device
    t = {k: v.to(dev) for k, v in syn.moe_tensors(syn.MOE_TINY, 2, seed=7).items()}
    fields = {f: t[f] for f in syn.MOE_WEIGHT_FIELDS}
    mixed = dict(fields, expert_gate=fields["expert_gate"].float())
    with pytest.raises(RuntimeError, match="expert_gate dtype mismatch"):
        mk.moe_decode(t["x"], mk.MoeWeights(**mixed), top_k=3, backend="persistent")
    with pytest.raises(RuntimeError, match="top_k must be in"):
        mk.moe_decode(t["x"], mk.MoeWeights(**fields), top_k=7)
    with pytest.raises(RuntimeError, match="must be contiguous"):
        mk.moe_decode(t["x"].t().contiguous().t(), mk.MoeWeights(**fields), top_k=3)
    with pytest.raises(RuntimeError, match="state must be float32"):
        mk.linear_attention_decode(mk.LinearAttentionInputs(
            q=torch.zeros(1, 2, 4, device=dev), k=torch.zeros(1, 2, 4, device=dev), v=torch.zeros(1, 2, 4, device=dev),
            state=torch.zeros(1, 2, 4, 4, device=dev, dtype=torch.float16)))
    with pytest.raises(RuntimeError, match="head_dim > 256"):
        mk.full_attention_decode(mk.FullAttentionInputs(
            q=torch.zeros(1, 2, 512, device=dev), k_cache=torch.zeros(1, 4, 2, 512, device=dev),
            v_cache=torch.zeros(1, 4, 2, 512, device=dev)))


def test_bounded_wait_reports_timeout_instead_of_hanging(cuda_device):
    """A barrier that can never complete gives up after its limit and raises the status word; the
    context stays usable and a re-initialised workspace works again."""
    import ctypes
    from mega_kernel_qwen36 import cabi

    lib = cabi.load()
    nbytes = lib.mk36_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device=cuda_device)
    stream = torch.cuda.current_stream().cuda_stream
    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    status = ctypes.c_int(-1)
    cabi.check(lib.mk36_workspace_status(ws.data_ptr(), stream, ctypes.byref(status)))
    assert status.value == 0
    cabi.check(lib.mk36_selftest_bounded_wait(ws.data_ptr(), nbytes, stream, 50))
    rc = lib.mk36_workspace_status(ws.data_ptr(), stream, ctypes.byref(status))
    assert rc == cabi.MK36_ERR_BARRIER_TIMEOUT and status.value == 901
    assert b"bounded device-side wait" in lib.mk36_last_error()
    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_workspace_status(ws.data_ptr(), stream, ctypes.byref(status)))
    assert status.value == 0
    assert float(torch.ones(4, device=cuda_device).sum()) == 4.0


def test_status_word_is_sticky_until_the_workspace_is_initialised_again(cuda_device):
    """After a bounded wait has given up (made on the host side: a barrier that expects an arrival
    nobody makes), every op queued on that workspace leaves at once: the status is still reported and
    the outputs are untouched.  Re-initialising the workspace makes the ops work again."""
    import ctypes

    from mega_kernel_qwen36 import cabi, synthetic as syn

    lib = cabi.load()
    dev = cuda_device
    nbytes = lib.mk36_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    status = ctypes.c_int(-1)

    d = {k: v.to(dev) for k, v in syn.dense_tensors(syn.DenseShape(256, 704), 3, seed=5).items()}
    d_out = torch.full_like(d["x"], 5.0)
    d_args = cabi.DenseFfnArgs(x=d["x"].data_ptr(), norm_weight=d["norm_weight"].data_ptr(), gate_weight=d["gate_weight"].data_ptr(),
                               up_weight=d["up_weight"].data_ptr(), down_weight=d["down_weight"].data_ptr(), out=d_out.data_ptr(),
                               partial_out=None, dtype=cabi.MK36_BF16, batch=3, hidden=256, intermediate=704, add_residual=1, eps=1e-6)
    m = {k: v.to(dev) for k, v in syn.moe_tensors(syn.MOE_35B_A3B, 1, 4).items()}
    m_out = torch.full_like(m["x"], 5.0)
    idx = torch.full((1, 8), -1, dtype=torch.int64, device=dev)
    rw = torch.full((1, 8), -1.0, dtype=torch.float32, device=dev)
    m_args = cabi.MoeArgs(x=m["x"].data_ptr(), norm_weight=m["norm_weight"].data_ptr(), router_weight=m["router_weight"].data_ptr(),
                          expert_gate=m["expert_gate"].data_ptr(), expert_up=m["expert_up"].data_ptr(), expert_down=m["expert_down"].data_ptr(),
                          shared_gate=m["shared_gate"].data_ptr(), shared_up=m["shared_up"].data_ptr(), shared_down=m["shared_down"].data_ptr(),
                          out=m_out.data_ptr(), indices=idx.data_ptr(), route_weights=rw.data_ptr(), partial_out=None, dtype=cabi.MK36_BF16,
                          batch=1, hidden=2048, experts=256, top_k=8, intermediate=512, shared_intermediate=512, expert_base=0,
                          local_experts=256, add_residual=1, eps=1e-6)
    t = {k: v.to(dev) for k, v in syn.attention_tensors(1, 16, 2, 256, 1024, seed=2).items()}
    a_out = torch.full_like(t["q"], 5.0)
    a_args = cabi.AttentionArgs(q=t["q"].data_ptr(), k_cache=t["k_cache"].data_ptr(), v_cache=t["v_cache"].data_ptr(), out=a_out.data_ptr(),
                                dtype=cabi.MK36_BF16, batch=1, query_heads=16, kv_heads=2, head_dim=256, seq_len=1024, scale=1.0 / 16)

    pj = {k: v.to(dev) for k, v in syn.projection_tensors(2048, 1536, 2, seed=9).items()}
    p_out = torch.full((2, 1536), 5.0, dtype=torch.bfloat16, device=dev)
    p_best = torch.full((2,), -7, dtype=torch.int64, device=dev)
    p_args = cabi.LinearArgs(x=pj["x"].data_ptr(), norm_weight=pj["norm_weight"].data_ptr(), weight=pj["weight"].data_ptr(),
                             residual=pj["residual"].data_ptr(), out=p_out.data_ptr(), argmax=p_best.data_ptr(), dtype=cabi.MK36_BF16,
                             batch=2, in_features=2048, out_features=1536, eps=1e-6)

    cabi.check(lib.mk36_selftest_bounded_wait(ws.data_ptr(), nbytes, stream, 20))
    cabi.check(lib.mk36_dense_ffn_decode(d_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_moe_decode(m_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_full_attention_decode(a_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_linear_decode(p_args, ws.data_ptr(), nbytes, stream))
    rc = lib.mk36_workspace_status(ws.data_ptr(), stream, ctypes.byref(status))
    assert rc == cabi.MK36_ERR_BARRIER_TIMEOUT and status.value == 901, (rc, status.value)
    for name, out in (("dense", d_out), ("moe", m_out), ("attention", a_out), ("projection", p_out)):
        assert bool((out == 5.0).all()), f"{name}: an op queued behind a timeout wrote its output"
    assert bool((p_best == -7).all())

    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_dense_ffn_decode(d_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_moe_decode(m_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_full_attention_decode(a_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_linear_decode(p_args, ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_workspace_status(ws.data_ptr(), stream, ctypes.byref(status)))
    assert status.value == 0
    assert bool((p_best >= 0).all()) and bool((p_best < 1536).all())
    for name, out in (("dense", d_out), ("moe", m_out), ("attention", a_out), ("projection", p_out)):
        assert torch.isfinite(out.float()).all() and not bool((out == 5.0).all()), name


def test_c_abi_direct_call_matches_extension(cuda_device):
    """The same kernel through ctypes (raw pointers, own workspace) and through the extension."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import cabi, synthetic as syn

    lib = cabi.load()
    dev = cuda_device
    t = {k: v.to(dev) for k, v in syn.dense_tensors(syn.DenseShape(256, 704), 3, seed=5).items()}
    expect = mk.dense_ffn_decode(t["x"], mk.DenseFfnWeights(*[t[f] for f in syn.DENSE_WEIGHT_FIELDS]))
    out = torch.empty_like(t["x"])
    args = cabi.DenseFfnArgs(x=t["x"].data_ptr(), norm_weight=t["norm_weight"].data_ptr(), gate_weight=t["gate_weight"].data_ptr(),
                             up_weight=t["up_weight"].data_ptr(), down_weight=t["down_weight"].data_ptr(), out=out.data_ptr(),
                             partial_out=None, dtype=cabi.MK36_BF16, batch=3, hidden=256, intermediate=704, add_residual=1, eps=1e-6)
    nbytes = lib.mk36_workspace_bytes()
    ws = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream().cuda_stream
    cabi.check(lib.mk36_workspace_init(ws.data_ptr(), nbytes, stream))
    cabi.check(lib.mk36_dense_ffn_decode(args, ws.data_ptr(), nbytes, stream))
    torch.cuda.synchronize()
    assert torch.equal(out, expect)
    # argument errors come back as status codes with a message, not as crashes
    args.hidden = 0
    assert lib.mk36_dense_ffn_decode(args, ws.data_ptr(), nbytes, stream) == cabi.MK36_ERR_INVALID_ARG
    assert b"sizes must be positive" in lib.mk36_last_error()
    args.hidden = 256
    assert lib.mk36_dense_ffn_decode(args, None, 0, stream) == cabi.MK36_ERR_WORKSPACE


LINEAR_CASES = [
    # batch, in_features, out_features, dtype, norm, residual
    (1, 2048, 5120, torch.bfloat16, True, False),    # q | k | v projection of the 35B-A3B attention layer
    (1, 4096, 2048, torch.bfloat16, False, True),    # attention output projection + residual
    (1, 5120, 1024, torch.bfloat16, True, True),     # 27B hidden size: three rows per 32 KB chunk
    (2, 2048, 1000, torch.float16, True, True),      # out_features not a multiple of the rows per chunk
    (3, 256, 77, torch.bfloat16, True, False),       # three tokens run as a group of four; few chunks
    (5, 1024, 4099, torch.float16, False, False),
    (8, 2048, 5120, torch.bfloat16, True, True),
    (8, 4096, 2048, torch.bfloat16, False, True),
]


@pytest.mark.parametrize("batch,k,n,dtype,norm,residual", LINEAR_CASES, ids=lambda v: str(v).replace("torch.", ""))
def test_linear_decode_matches_oracle(batch, k, n, dtype, norm, residual, cuda_device):
    """Decode-time projection (fused RMSNorm, residual) against the CPU oracle and its fp64 evaluation."""
    import mega_kernel_qwen36 as mk
    from oracle import decode_oracle as oracle
    from mega_kernel_qwen36 import synthetic as syn

    t = syn.projection_tensors(k, n, batch, seed=31 + batch, dtype=dtype, norm=norm, residual=residual)
    d = {name: v.to(cuda_device) for name, v in t.items()}
    got = mk.linear_decode(d["x"], d["weight"], norm_weight=d.get("norm_weight"), residual=d.get("residual")).cpu()
    ref = oracle.linear_decode(t["x"], t["weight"], norm_weight=t.get("norm_weight"), residual=t.get("residual"))
    assert got.dtype == dtype and got.shape == (batch, n)
    assert_output_parity(got, ref, what=f"linear_decode {batch}x{k}->{n}")
    f64 = oracle.linear_decode_f64(t["x"], t["weight"], norm_weight=t.get("norm_weight"), residual=t.get("residual"))
    assert rel_l2(got.double(), f64) <= 5e-3
    # the same call twice gives the same bits (no atomics on the data path)
    again = mk.linear_decode(d["x"], d["weight"], norm_weight=d.get("norm_weight"), residual=d.get("residual")).cpu()
    assert torch.equal(got, again)


@pytest.mark.parametrize("batch,k,n", [(3, 256, 77), (5, 1024, 4099), (8, 2048, 5120)])
def test_linear_decode_plain_fma_path_for_several_tokens(batch, k, n, cuda_device):
    """Three to eight tokens normally run on tensor-core tiles; the plain-FMA path (four rows x four tokens per
    warp), which also serves inner dimensions that are not a multiple of 256, must give the same answer."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import cabi, synthetic as syn
    from oracle import decode_oracle as oracle

    t = syn.projection_tensors(k, n, batch, seed=77, norm=True, residual=True)
    d = {name: v.to(cuda_device) for name, v in t.items()}
    lib = cabi.load()
    tiles, best_tiles = mk.linear_decode(d["x"], d["weight"], norm_weight=d["norm_weight"], residual=d["residual"], return_argmax=True)
    cabi.check(lib.mk36_set_option(b"linear_mma", 0))
    try:
        plain, best_plain = mk.linear_decode(d["x"], d["weight"], norm_weight=d["norm_weight"], residual=d["residual"], return_argmax=True)
    finally:
        cabi.check(lib.mk36_set_option(b"linear_mma", 3))
    ref = oracle.linear_decode(t["x"], t["weight"], norm_weight=t["norm_weight"], residual=t["residual"])
    assert_output_parity(plain.cpu(), ref, what="plain-FMA path")
    assert_output_parity(tiles.cpu(), ref, what="tensor-core path")
    for out, best in ((tiles, best_tiles), (plain, best_plain)):
        row_max = out.float().max(dim=-1, keepdim=True).values
        assert torch.equal(best, (out.float() == row_max).float().argmax(dim=-1))
    # inner dimension not a multiple of 256: served by the plain path whatever the switch says
    t2 = syn.projection_tensors(k + 8, n, batch, seed=78, norm=True, residual=False)
    d2 = {name: v.to(cuda_device) for name, v in t2.items()}
    got = mk.linear_decode(d2["x"], d2["weight"], norm_weight=d2["norm_weight"]).cpu()
    assert_output_parity(got, oracle.linear_decode(t2["x"], t2["weight"], norm_weight=t2["norm_weight"]), what="odd inner dimension")


@pytest.mark.parametrize("batch,n", [(1, 30_001), (4, 248_320), (7, 9_000)])
def test_linear_decode_argmax_is_the_argmax_of_the_stored_row(batch, n, cuda_device):
    """LM-head use: the arg-max comes from the same launch; lowest index among equal (rounded) values."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    k = 2048 if n > 100_000 else 512
    t = syn.projection_tensors(k, n, batch, seed=5, dtype=torch.bfloat16, norm=True, residual=False)
    d = {name: v.to(cuda_device) for name, v in t.items()}
    for _ in range(2):  # the arg-max slots of the workspace must be clean again after a call
        out, best = mk.linear_decode(d["x"], d["weight"], norm_weight=d["norm_weight"], return_argmax=True)
        assert best.dtype == torch.int64 and best.shape == (batch,)
        # torch.argmax does not promise the first index among equals; max + first match does
        row_max = out.float().max(dim=-1, keepdim=True).values
        first = (out.float() == row_max).float().argmax(dim=-1)
        assert torch.equal(best, first), (best, first)
    # rows whose top values tie after rounding: duplicate the best row of the weight further up
    w = d["weight"].clone()
    top = int(best[0])
    later = (top + 1234) % n
    w[later] = w[top]
    out, best2 = mk.linear_decode(d["x"], w, norm_weight=d["norm_weight"], return_argmax=True)
    assert int(best2[0]) == min(top, later)


def test_linear_decode_refuses_what_it_does_not_take(cuda_device):
    import mega_kernel_qwen36 as mk

    x = torch.zeros(9, 256, dtype=torch.bfloat16, device=cuda_device)
    w = torch.zeros(64, 256, dtype=torch.bfloat16, device=cuda_device)
    with pytest.raises(RuntimeError, match="at most 8 tokens"):
        mk.linear_decode(x, w)
    with pytest.raises(RuntimeError, match="multiple of 8"):
        mk.linear_decode(x[:1, :250].contiguous(), w[:, :250].contiguous())
    with pytest.raises(RuntimeError, match="bf16 or f16|dtype"):
        mk.linear_decode(x[:1].float(), w.float())


@pytest.mark.parametrize("batch,rope", [(1, True), (2, False)])
def test_attention_block_with_projections_in_decode_layer(batch, rope, cuda_device):
    """Full-attention layer at the 35B-A3B head geometry (16 query heads, 2 KV heads, head_dim 256: heads x
    dim != hidden): fused norm + q|k|v projection, rotary on the new query and key, cache append, attention,
    output projection + residual, then the MoE - against the same composition of the CPU oracle."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn
    from oracle import decode_oracle as oracle

    H, hq, hkv, d, tmax, pos = 2048, 16, 2, 256, 384, 300
    dev = cuda_device
    moe_t = syn.moe_tensors(syn.MOE_35B_A3B, batch, seed=41)
    hidden = moe_t["x"]
    qkv = syn.projection_tensors(H, (hq + 2 * hkv) * d, batch, seed=42, norm=True, residual=False)
    outp = syn.projection_tensors(hq * d, H, batch, seed=43, norm=False, residual=False)
    cache = syn.attention_tensors(batch, hq, hkv, d, tmax, seed=44)
    cos = sin = None
    if rope:
        ang = torch.arange(32, dtype=torch.float32) * 0.37 + 0.1
        cos, sin = torch.cat((ang.cos(), ang.cos())), torch.cat((ang.sin(), ang.sin()))
    block = mk.AttentionBlockInputs(
        input_norm_weight=qkv["norm_weight"].to(dev), qkv_weight=qkv["weight"].to(dev), out_weight=outp["weight"].to(dev),
        k_cache=cache["k_cache"].to(dev), v_cache=cache["v_cache"].to(dev), position=pos, query_heads=hq, kv_heads=hkv, head_dim=d,
        cos=cos, sin=sin, rotary_dim=64, scale=1.0 / 16)
    moe_w = mk.MoeWeights(*[moe_t[f].to(dev) for f in syn.MOE_WEIGHT_FIELDS])
    r = mk.decode_layer(3, hidden.to(dev), moe_w, top_k=8, attention_block=block)

    mid, attn, k_ref, v_ref = oracle.attention_block_decode(
        hidden, qkv["norm_weight"], qkv["weight"], outp["weight"], cache["k_cache"], cache["v_cache"], pos, hq, hkv, d,
        cos=cos, sin=sin, rotary_dim=64, scale=1.0 / 16)
    want, idx, _ = oracle.moe_decode(mid, *[moe_t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=8)
    assert_output_parity(r.attention_output.cpu(), attn, what="attention output")
    assert_output_parity(block.k_cache[:, pos].cpu(), k_ref[:, pos], what="appended key")
    assert_output_parity(block.v_cache[:, pos].cpu(), v_ref[:, pos], what="appended value")
    assert torch.equal(block.k_cache[:, :pos].cpu(), cache["k_cache"][:, :pos])
    if torch.equal(r.router_indices.cpu(), idx):  # a routing near-tie can flip an expert after three rounded stages
        assert_output_parity(r.hidden.cpu(), want, what="layer output")
    else:
        assert (r.router_indices.cpu() == idx).float().mean() >= 0.9
