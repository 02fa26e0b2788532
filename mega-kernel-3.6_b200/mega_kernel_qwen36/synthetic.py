"""Seeded synthetic inputs for the decode ops.

All tensors are drawn on the CPU from ``numpy.random.Generator(PCG64(seed))`` in a fixed order
and only then cast / moved, so that a CPU checker and the CUDA kernels see bit-identical values
on any machine with the same numpy.  Shapes and distributions follow the workloads the decode
layer is measured on: weights ~ N(0, 0.02), hidden states ~ N(0, 1), KV cache ~ N(0, 1),
recurrent state ~ N(0, 0.1), L2-normalised q/k for the recurrence.

The reference draws its test tensors with ``torch.randn`` (tests/test_reference.py:18-47,
benchmarks/bench_moe.py:29-43); only shapes, scales and dtypes are taken from there.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import numpy as np
import torch


def _rng(seed: int) -> np.random.Generator:
    return np.random.Generator(np.random.PCG64(seed))


def _normal(rng: np.random.Generator, shape, std: float = 1.0, mean: float = 0.0) -> torch.Tensor:
    arr = rng.standard_normal(size=shape, dtype=np.float32)
    if std != 1.0:
        arr *= np.float32(std)
    if mean != 0.0:
        arr += np.float32(mean)
    return torch.from_numpy(arr)


@dataclass(frozen=True)
class MoeShape:
    hidden: int
    experts: int
    top_k: int
    intermediate: int
    shared_intermediate: int


MOE_SMALL = MoeShape(hidden=256, experts=16, top_k=4, intermediate=128, shared_intermediate=128)
MOE_35B_A3B = MoeShape(hidden=2048, experts=256, top_k=8, intermediate=512, shared_intermediate=512)
MOE_TINY = MoeShape(hidden=16, experts=6, top_k=3, intermediate=12, shared_intermediate=12)


def moe_weights(
    shape: MoeShape,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    *,
    w_std: float = 0.02,
    norm_jitter: float = 0.0,
) -> Dict[str, torch.Tensor]:
    """The eight weight tensors of ``MoeWeights``, by field name.  They depend on the seed only,
    so one draw serves every batch size."""
    rng = _rng(seed)
    h, e, i, s = shape.hidden, shape.experts, shape.intermediate, shape.shared_intermediate
    out = {}
    if norm_jitter:
        out["norm_weight"] = _normal(rng, (h,), norm_jitter, 1.0).to(dtype)
    else:
        out["norm_weight"] = torch.ones(h, dtype=dtype)
    out["router_weight"] = _normal(rng, (e, h), w_std).to(dtype)
    out["expert_gate"] = _normal(rng, (e, i, h), w_std).to(dtype)
    out["expert_up"] = _normal(rng, (e, i, h), w_std).to(dtype)
    out["expert_down"] = _normal(rng, (e, h, i), w_std).to(dtype)
    out["shared_gate"] = _normal(rng, (s, h), w_std).to(dtype)
    out["shared_up"] = _normal(rng, (s, h), w_std).to(dtype)
    out["shared_down"] = _normal(rng, (h, s), w_std).to(dtype)
    return out


def hidden_states(batch: int, hidden: int, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                  *, x_std: float = 1.0) -> torch.Tensor:
    """x [batch, hidden] ~ N(0, x_std); its stream is separate from the weights' stream."""
    return _normal(_rng(seed + 1_000_003), (batch, hidden), x_std).to(dtype)


def moe_tensors(
    shape: MoeShape,
    batch: int,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    *,
    x_std: float = 1.0,
    w_std: float = 0.02,
    norm_jitter: float = 0.0,
) -> Dict[str, torch.Tensor]:
    """``x`` plus the weights of ``moe_weights``."""
    out = {"x": hidden_states(batch, shape.hidden, seed, dtype, x_std=x_std)}
    out.update(moe_weights(shape, seed, dtype, w_std=w_std, norm_jitter=norm_jitter))
    return out


MOE_WEIGHT_FIELDS = (
    "norm_weight", "router_weight", "expert_gate", "expert_up", "expert_down",
    "shared_gate", "shared_up", "shared_down",
)


@dataclass(frozen=True)
class DenseShape:
    hidden: int
    intermediate: int


DENSE_27B = DenseShape(hidden=5120, intermediate=17408)
DENSE_TINY = DenseShape(hidden=16, intermediate=24)

DENSE_WEIGHT_FIELDS = ("norm_weight", "gate_weight", "up_weight", "down_weight")


def dense_weights(
    shape: DenseShape,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    *,
    w_std: float = 0.02,
    norm_jitter: float = 0.0,
) -> Dict[str, torch.Tensor]:
    rng = _rng(seed)
    h, i = shape.hidden, shape.intermediate
    out = {}
    if norm_jitter:
        out["norm_weight"] = _normal(rng, (h,), norm_jitter, 1.0).to(dtype)
    else:
        out["norm_weight"] = torch.ones(h, dtype=dtype)
    out["gate_weight"] = _normal(rng, (i, h), w_std).to(dtype)
    out["up_weight"] = _normal(rng, (i, h), w_std).to(dtype)
    out["down_weight"] = _normal(rng, (h, i), w_std).to(dtype)
    return out


def dense_tensors(
    shape: DenseShape,
    batch: int,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    *,
    x_std: float = 1.0,
    w_std: float = 0.02,
    norm_jitter: float = 0.0,
) -> Dict[str, torch.Tensor]:
    out = {"x": hidden_states(batch, shape.hidden, seed, dtype, x_std=x_std)}
    out.update(dense_weights(shape, seed, dtype, w_std=w_std, norm_jitter=norm_jitter))
    return out


def attention_tensors(
    batch: int,
    query_heads: int,
    kv_heads: int,
    head_dim: int,
    seq_len: int,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
    *,
    std: float = 1.0,
) -> Dict[str, torch.Tensor]:
    """q [B,Hq,D]; k_cache, v_cache [B,T,Hkv,D] (token-major, heads interleaved)."""
    rng = _rng(seed)
    return {
        "q": _normal(rng, (batch, query_heads, head_dim), std).to(dtype),
        "k_cache": _normal(rng, (batch, seq_len, kv_heads, head_dim), std).to(dtype),
        "v_cache": _normal(rng, (batch, seq_len, kv_heads, head_dim), std).to(dtype),
    }


def linear_state(batch: int, value_heads: int, key_dim: int, value_dim: int, seed: int = 0,
                 std: float = 0.1) -> torch.Tensor:
    return _normal(_rng(seed + 7919), (batch, value_heads, key_dim, value_dim), std)


def linear_step_stream(
    batch: int,
    key_heads: int,
    value_heads: int,
    key_dim: int,
    value_dim: int,
    steps: int,
    seed: int = 0,
    dtype: torch.dtype = torch.bfloat16,
):
    """Yields ``steps`` dicts {q,k,v,g,beta} from one generator stream: q,k ~ N(0,1) then
    L2-normalised over the key dim, v ~ N(0,1), g = sigmoid(N(0,1)) and beta = sigmoid(N(0,1))
    per (batch, value head)."""
    rng = _rng(seed)
    for _ in range(steps):
        q = _normal(rng, (batch, key_heads, key_dim))
        k = _normal(rng, (batch, key_heads, key_dim))
        # normalise in float64 so that the rounded result does not depend on the host's
        # summation order
        q = (q.double() / q.double().pow(2).sum(dim=-1, keepdim=True).sqrt()).float()
        k = (k.double() / k.double().pow(2).sum(dim=-1, keepdim=True).sqrt()).float()
        v = _normal(rng, (batch, value_heads, value_dim))
        g = torch.sigmoid(_normal(rng, (batch, value_heads)))
        beta = torch.sigmoid(_normal(rng, (batch, value_heads)))
        yield {"q": q.to(dtype), "k": k.to(dtype), "v": v.to(dtype), "g": g, "beta": beta}


# ---------------------------------------------------------------------------------------------
# Algorithmic bytes: every distinct byte that has to cross HBM once per decode step.
# ---------------------------------------------------------------------------------------------
def moe_algorithmic_bytes(shape: MoeShape, batch: int, distinct_experts: int, elem: int = 2) -> int:
    h, e, k = shape.hidden, shape.experts, shape.top_k
    i, s = shape.intermediate, shape.shared_intermediate
    return (distinct_experts * 3 * i * h * elem + 3 * s * h * elem + e * h * elem + h * elem
            + 2 * batch * h * elem + batch * k * 12)


def dense_algorithmic_bytes(shape: DenseShape, batch: int, elem: int = 2) -> int:
    return 3 * shape.intermediate * shape.hidden * elem + shape.hidden * elem + 2 * batch * shape.hidden * elem


def attention_algorithmic_bytes(batch: int, query_heads: int, kv_heads: int, head_dim: int,
                                seq_len: int, elem: int = 2) -> int:
    return batch * (2 * seq_len * kv_heads * head_dim * elem + 2 * query_heads * head_dim * elem)


def linear_algorithmic_bytes(batch: int, key_heads: int, value_heads: int, key_dim: int,
                             value_dim: int, elem: int = 2) -> int:
    state = 2 * batch * value_heads * key_dim * value_dim * 4
    vecs = batch * (2 * key_heads * key_dim + 2 * value_heads * value_dim) * elem
    return state + vecs


# --------------------------------------------------------------------------------------------
# Decode-time projections (the q/k/v projection, the attention output projection, the LM head)
# --------------------------------------------------------------------------------------------
# Qwen3.6-35B-A3B full-attention layer: hidden 2048; 16 query heads, 2 KV heads, head_dim 256.
QKV_35B = (2048, 16 * 256 + 2 * 2 * 256)   # (in_features, out_features): hidden -> q | k | v
OUT_PROJ_35B = (16 * 256, 2048)             # attention output -> hidden, plus residual
LM_HEAD_35B = (2048, 248_320)               # hidden -> vocabulary


def projection_tensors(in_features: int, out_features: int, batch: int, seed: int = 0, dtype: torch.dtype = torch.bfloat16,
                       *, x_std: float = 1.0, w_std: float = 0.02, norm: bool = True, residual: bool = True,
                       norm_jitter: float = 0.05) -> Dict[str, torch.Tensor]:
    """x [batch, in]; weight [out, in]; optionally norm_weight [in] ~ N(1, jitter) and residual [batch, out]."""
    rng = _rng(seed)
    out = {"x": hidden_states(batch, in_features, seed, dtype, x_std=x_std),
           "weight": _normal(rng, (out_features, in_features), w_std).to(dtype)}
    if norm:
        out["norm_weight"] = _normal(rng, (in_features,), norm_jitter, 1.0).to(dtype)
    if residual:
        out["residual"] = _normal(rng, (batch, out_features), x_std).to(dtype)
    return out


def projection_algorithmic_bytes(in_features: int, out_features: int, batch: int, *, norm: bool, residual: bool, elem: int = 2) -> int:
    n = out_features * in_features * elem + batch * in_features * elem + batch * out_features * elem
    if norm:
        n += in_features * elem
    if residual:
        n += batch * out_features * elem
    return n
