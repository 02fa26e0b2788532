"""The seeded cases whose reference outputs are stored under tests/golden/.

Each case rebuilds its inputs from a seed (mega_kernel_qwen36.synthetic, numpy PCG64) and names
the op it feeds.  ``tests/golden/make_golden.py`` ran the reference's own ``reference.py`` on
these inputs and stored the outputs; ``tests/test_golden.py`` re-runs the CPU oracle on them and
``tests/test_gpu_parity.py`` the CUDA kernels.
"""

from __future__ import annotations

from typing import Callable, Dict, NamedTuple

import torch

from mega_kernel_qwen36 import synthetic as syn


class Case(NamedTuple):
    name: str
    op: str                      # moe | dense | attention | linear
    build: Callable[[], Dict]    # inputs and keyword arguments
    heavy: bool = False          # full model dimensions (seconds of CPU time)


def _moe(shape, batch, seed, dtype, top_k=None, **kw):
    def build():
        t = syn.moe_tensors(shape, batch, seed, dtype, **kw)
        return {"tensors": t, "top_k": top_k or shape.top_k}
    return build


def _dense(shape, batch, seed, dtype, **kw):
    return lambda: {"tensors": syn.dense_tensors(shape, batch, seed, dtype, **kw)}


def _attn(batch, hq, hkv, d, t, seed, dtype, std=1.0, scale=None):
    return lambda: {"tensors": syn.attention_tensors(batch, hq, hkv, d, t, seed, dtype, std=std), "scale": scale}


def _linear(batch, hk, hv, dk, dv, steps, seed, dtype, decay):
    def build():
        return {
            "state": syn.linear_state(batch, hv, dk, dv, seed),
            "steps": list(syn.linear_step_stream(batch, hk, hv, dk, dv, steps, seed, dtype)),
            "decay": decay,
            "expand": hv // hk,
        }
    return build


BF16, F32, F16 = torch.bfloat16, torch.float32, torch.float16

CASES = [
    # --- MoE -------------------------------------------------------------------------------
    Case("moe_small_f32_b1", "moe", _moe(syn.MOE_SMALL, 1, 0, F32)),
    Case("moe_small_f32_b1_normjitter", "moe", _moe(syn.MOE_SMALL, 1, 0, F32, norm_jitter=0.02)),
    Case("moe_small_bf16_b3", "moe", _moe(syn.MOE_SMALL, 3, 1, BF16)),
    Case("moe_small_f16_b2", "moe", _moe(syn.MOE_SMALL, 2, 2, F16)),
    Case("moe_tiny_f32_b2", "moe", _moe(syn.MOE_TINY, 2, 7, F32, x_std=0.08, w_std=0.08, norm_jitter=0.08)),
    Case("moe_tiny_bf16_b8", "moe", _moe(syn.MOE_TINY, 8, 7, BF16, x_std=0.08, w_std=0.08, norm_jitter=0.08)),
    Case("moe_tiny_bf16_b11", "moe", _moe(syn.MOE_TINY, 11, 8, BF16, x_std=1.0, w_std=0.3, norm_jitter=0.08)),
    Case("moe_35b_bf16_b1_s0", "moe", _moe(syn.MOE_35B_A3B, 1, 0, BF16), heavy=True),
    Case("moe_35b_bf16_b2_s0", "moe", _moe(syn.MOE_35B_A3B, 2, 0, BF16), heavy=True),
    Case("moe_35b_bf16_b4_s0", "moe", _moe(syn.MOE_35B_A3B, 4, 0, BF16), heavy=True),
    Case("moe_35b_bf16_b8_s0", "moe", _moe(syn.MOE_35B_A3B, 8, 0, BF16), heavy=True),
    Case("moe_35b_bf16_b1_s1", "moe", _moe(syn.MOE_35B_A3B, 1, 1, BF16), heavy=True),
    Case("moe_35b_bf16_b2_s1", "moe", _moe(syn.MOE_35B_A3B, 2, 1, BF16), heavy=True),
    Case("moe_35b_bf16_b4_s1", "moe", _moe(syn.MOE_35B_A3B, 4, 1, BF16), heavy=True),
    Case("moe_35b_bf16_b8_s1", "moe", _moe(syn.MOE_35B_A3B, 8, 1, BF16), heavy=True),
    Case("moe_35b_bf16_b1_s2", "moe", _moe(syn.MOE_35B_A3B, 1, 2, BF16), heavy=True),
    Case("moe_35b_bf16_b2_s2", "moe", _moe(syn.MOE_35B_A3B, 2, 2, BF16), heavy=True),
    Case("moe_35b_bf16_b4_s2", "moe", _moe(syn.MOE_35B_A3B, 4, 2, BF16), heavy=True),
    Case("moe_35b_bf16_b8_s2", "moe", _moe(syn.MOE_35B_A3B, 8, 2, BF16), heavy=True),
    # --- dense FFN -------------------------------------------------------------------------
    Case("dense_tiny_f32_b2", "dense", _dense(syn.DENSE_TINY, 2, 23, F32, x_std=0.08, w_std=0.08, norm_jitter=0.08)),
    Case("dense_tiny_bf16_b8", "dense", _dense(syn.DENSE_TINY, 8, 23, BF16, x_std=0.08, w_std=0.08, norm_jitter=0.08)),
    Case("dense_mid_bf16_b3", "dense", _dense(syn.DenseShape(256, 704), 3, 5, BF16)),
    Case("dense_mid_f16_b1", "dense", _dense(syn.DenseShape(256, 704), 1, 6, F16)),
    Case("dense_27b_bf16_b1", "dense", _dense(syn.DENSE_27B, 1, 0, BF16), heavy=True),
    Case("dense_27b_bf16_b8", "dense", _dense(syn.DENSE_27B, 8, 0, BF16), heavy=True),
    # --- full attention --------------------------------------------------------------------
    Case("attn_tiny_bf16_t1", "attention", _attn(2, 4, 2, 32, 1, 17, BF16, std=0.1)),
    Case("attn_tiny_bf16_t128", "attention", _attn(2, 4, 2, 32, 128, 17, BF16, std=0.1)),
    Case("attn_tiny_bf16_t4096", "attention", _attn(2, 4, 2, 32, 4096, 17, BF16, std=0.1)),
    Case("attn_tiny_f32_t9", "attention", _attn(2, 4, 2, 16, 9, 11, F32)),
    Case("attn_odd_bf16_t777", "attention", _attn(3, 6, 2, 80, 777, 3, BF16)),
    Case("attn_27b_bf16_t1000", "attention", _attn(1, 24, 4, 256, 1000, 4, BF16)),
    Case("attn_35b_bf16_t4096", "attention", _attn(1, 16, 2, 256, 4096, 0, BF16, scale=1.0 / 16)),
    Case("attn_35b_bf16_t8192", "attention", _attn(1, 16, 2, 256, 8192, 0, BF16, scale=1.0 / 16), heavy=True),
    Case("attn_35b_bf16_t16384", "attention", _attn(1, 16, 2, 256, 16384, 0, BF16, scale=1.0 / 16), heavy=True),
    Case("attn_35b_bf16_t32768", "attention", _attn(1, 16, 2, 256, 32768, 0, BF16, scale=1.0 / 16), heavy=True),
    Case("attn_35b_bf16_b2_t2500", "attention", _attn(2, 16, 2, 256, 2500, 9, BF16)),
    # --- linear attention (64 consecutive steps; scalar decay; q/k expanded to the value heads) --
    Case("linear_tiny_bf16", "linear", _linear(2, 3, 3, 8, 10, 3, 19, BF16, 0.92)),
    Case("linear_tiny_f32", "linear", _linear(2, 3, 3, 5, 7, 2, 13, F32, 0.9)),
    Case("linear_35b_bf16_b1", "linear", _linear(1, 16, 32, 128, 128, 64, 0, BF16, 0.9), heavy=True),
    Case("linear_35b_bf16_b8", "linear", _linear(8, 16, 32, 128, 128, 64, 0, BF16, 0.9), heavy=True),
]

CASES_BY_NAME = {c.name: c for c in CASES}

# Entries kept from the recurrent state in the fixtures: every STATE_STRIDE-th row and column.
STATE_STRIDE = 16


def checksum(t: torch.Tensor) -> float:
    """Order-independent fingerprint of an input tensor (guards against a different RNG stream)."""
    return float(t.double().sum()) + float(t.double().abs().sum()) * 1e-3
