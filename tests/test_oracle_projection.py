"""The oracle's decode-time projection and attention block (CPU only).

The reference has no implementation of these (its planner names the tasks, its ops start from q and the
caches), so there is nothing to pin them to: the checks here are the fp64 evaluation of the same formulas
and the identities the composition must satisfy.
"""

import torch

from mega_kernel_qwen36 import synthetic as syn
from oracle import decode_oracle as oracle
from parity import rel_l2


def test_linear_decode_against_fp64_and_its_parts():
    t = syn.projection_tensors(512, 300, 3, seed=2, norm=True, residual=True)
    got = oracle.linear_decode(t["x"], t["weight"], norm_weight=t["norm_weight"], residual=t["residual"])
    f64 = oracle.linear_decode_f64(t["x"], t["weight"], norm_weight=t["norm_weight"], residual=t["residual"])
    assert got.dtype == torch.bfloat16 and got.shape == (3, 300)
    assert rel_l2(got.double(), f64) <= 4e-3
    # without norm and residual it is torch's linear on the fp32 copies, rounded once
    plain = oracle.linear_decode(t["x"], t["weight"])
    assert torch.equal(plain, torch.nn.functional.linear(t["x"].float(), t["weight"].float()).to(torch.bfloat16))
    # the fused norm is rms_norm followed by the plain projection
    xn = oracle.rms_norm(t["x"], t["norm_weight"], 1e-6)
    assert torch.equal(oracle.linear_decode(t["x"], t["weight"], norm_weight=t["norm_weight"]), oracle.linear_decode(xn, t["weight"]))


def test_attention_block_is_the_composition_of_its_parts():
    b, h, hq, hkv, d, tmax, pos = 2, 64, 4, 2, 16, 12, 7
    hidden = syn.hidden_states(b, h, seed=1)
    qkv = syn.projection_tensors(h, (hq + 2 * hkv) * d, b, seed=2, norm=True, residual=False, w_std=0.2)
    outp = syn.projection_tensors(hq * d, h, b, seed=3, norm=False, residual=False, w_std=0.2)
    cache = syn.attention_tensors(b, hq, hkv, d, tmax, seed=4)
    out, attn, k2, v2 = oracle.attention_block_decode(hidden, qkv["norm_weight"], qkv["weight"], outp["weight"], cache["k_cache"],
                                                       cache["v_cache"], pos, hq, hkv, d)
    assert out.shape == hidden.shape and attn.shape == (b, hq, d)
    assert torch.equal(k2[:, :pos], cache["k_cache"][:, :pos]) and torch.equal(k2[:, pos + 1 :], cache["k_cache"][:, pos + 1 :])
    proj = oracle.linear_decode(hidden, qkv["weight"], norm_weight=qkv["norm_weight"])
    assert torch.equal(k2[:, pos].reshape(b, -1), proj[:, hq * d : (hq + hkv) * d])
    assert torch.equal(v2[:, pos].reshape(b, -1), proj[:, (hq + hkv) * d :])
    again = oracle.full_attention_decode(proj[:, : hq * d].reshape(b, hq, d), k2[:, : pos + 1], v2[:, : pos + 1])
    assert torch.equal(attn, again)
    assert torch.equal(out, oracle.linear_decode(attn.reshape(b, hq * d), outp["weight"], residual=hidden))
