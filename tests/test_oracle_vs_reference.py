"""The CPU oracle against the reference's reference.py imported live from a reference checkout.

Runs only where the environment variable MK36_REFERENCE_ROOT names such a checkout; elsewhere
the committed fixtures (tests/test_golden.py) carry the same pin.  Seeds here differ from the
fixture seeds on purpose.
"""

import importlib.util
import os
from pathlib import Path

import pytest
import torch

from mega_kernel_qwen36 import synthetic as syn
from oracle import decode_oracle as oracle

REF_ROOT = os.environ.get("MK36_REFERENCE_ROOT")
REF_FILE = Path(REF_ROOT) / "mega_kernel_qwen36" / "reference.py" if REF_ROOT else None

pytestmark = pytest.mark.skipif(REF_FILE is None or not REF_FILE.exists(),
                                reason="MK36_REFERENCE_ROOT does not name a reference checkout")


@pytest.fixture(scope="module")
def ref():
    spec = importlib.util.spec_from_file_location("mk36_upstream_reference_live", REF_FILE)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
@pytest.mark.parametrize("batch,seed", [(1, 100), (5, 101)])
def test_moe(ref, dtype, batch, seed):
    t = syn.moe_tensors(syn.MoeShape(128, 24, 5, 96, 64), batch, seed, dtype, norm_jitter=0.05)
    w = [t[f] for f in syn.MOE_WEIGHT_FIELDS]
    for res in (True, False):
        a = oracle.moe_decode(t["x"], *w, top_k=5, add_residual=res)
        b = ref.moe_decode_reference(t["x"], *w, top_k=5, add_residual=res)
        for x, y in zip(a, b):
            assert x.dtype == y.dtype and torch.equal(x, y)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dense(ref, dtype):
    t = syn.dense_tensors(syn.DenseShape(192, 320), 4, 102, dtype, norm_jitter=0.05)
    w = [t[f] for f in syn.DENSE_WEIGHT_FIELDS]
    assert torch.equal(oracle.dense_ffn_decode(t["x"], *w), ref.dense_ffn_decode_reference(t["x"], *w))
    assert torch.equal(oracle.rms_norm(t["x"], w[0], 1e-5), ref.rms_norm(t["x"], w[0], 1e-5))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seq", [1, 37, 600])
def test_attention_and_rope(ref, dtype, seq):
    t = syn.attention_tensors(2, 6, 3, 48, seq, 103, dtype)
    assert torch.equal(oracle.full_attention_decode(**t), ref.full_attention_decode_reference(**t))
    assert torch.equal(oracle.full_attention_decode(**t, scale=0.3), ref.full_attention_decode_reference(**t, scale=0.3))
    ang = torch.linspace(0, 2, 8).repeat(2)
    a = oracle.apply_partial_rope(t["q"], t["k_cache"], torch.cos(ang), torch.sin(ang), 16)
    b = ref.apply_partial_rope(t["q"], t["k_cache"], torch.cos(ang), torch.sin(ang), 16)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    same = oracle.apply_partial_rope(t["q"], t["k_cache"], None, None, 16)
    assert same[0] is t["q"] and same[1] is t["k_cache"]


def test_linear_attention(ref):
    state = syn.linear_state(2, 6, 16, 24, seed=104)
    s_a = s_b = state
    for step in syn.linear_step_stream(2, 6, 6, 16, 24, steps=5, seed=104):
        o_a, s_a = oracle.linear_attention_decode(step["q"], step["k"], step["v"], s_a, decay=0.83)
        o_b, s_b = ref.linear_attention_decode_reference(step["q"], step["k"], step["v"], s_b, decay=0.83)
        assert torch.equal(o_a, o_b) and torch.equal(s_a, s_b)


def test_per_head_variant_reduces_to_reference(ref):
    """With one decay for all heads and beta = 1 the per-head form is the reference recurrence."""
    state = syn.linear_state(2, 4, 8, 8, seed=105)
    step = next(syn.linear_step_stream(2, 2, 4, 8, 8, steps=1, seed=105))
    decay = torch.full((2, 4), 0.7)
    o_a, s_a = oracle.linear_attention_decode_per_head(step["q"], step["k"], step["v"], state, decay, None)
    q = step["q"].repeat_interleave(2, dim=1)
    k = step["k"].repeat_interleave(2, dim=1)
    o_b, s_b = ref.linear_attention_decode_reference(q, k, step["v"], state, decay=0.7)
    torch.testing.assert_close(s_a, s_b, rtol=0, atol=0)
    torch.testing.assert_close(o_a.float(), o_b.float(), rtol=1e-2, atol=1e-3)
