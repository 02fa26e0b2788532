"""Decode-layer operators backed by the sm_100a kernels.

Drop-in for the decode part of the reference's ``mega_kernel_qwen36/ops.py``: the same
dataclasses (ops.py:38-75, 129-136), the same functions, keywords and defaults
(``moe_decode`` ops.py:277-320, ``dense_ffn_decode`` ops.py:323-364, ``full_attention_decode``
ops.py:367-374, ``linear_attention_decode`` ops.py:377-386, ``decode_layer`` ops.py:701-748,
``extension_available`` ops.py:145-146) and the same ``backend=`` names with the same
``ValueError`` for unknown ones.

Differences, all deliberate:
  * every CUDA backend name selects the one hand-written kernel for that op; there is no
    grouped-torch, Triton or cuBLAS path;
  * there is no CPU computation in this package.  CPU tensors, ``backend="reference"`` and a
    missing extension raise ``RuntimeError`` instead of silently running PyTorch code.
"""

from __future__ import annotations

import math
from dataclasses import dataclass
from typing import Optional, Tuple

import torch

from .config import qwen36_layer_type

_IMPORT_ERROR: Optional[BaseException] = None
try:
    from . import _C  # type: ignore[attr-defined]
except Exception as exc:  # the extension has not been built for this interpreter
    _C = None
    _IMPORT_ERROR = exc


@dataclass(frozen=True)
class MoeWeights:
    norm_weight: torch.Tensor
    router_weight: torch.Tensor
    expert_gate: torch.Tensor
    expert_up: torch.Tensor
    expert_down: torch.Tensor
    shared_gate: torch.Tensor
    shared_up: torch.Tensor
    shared_down: torch.Tensor


@dataclass(frozen=True)
class DenseFfnWeights:
    norm_weight: torch.Tensor
    gate_weight: torch.Tensor
    up_weight: torch.Tensor
    down_weight: torch.Tensor


@dataclass(frozen=True)
class FullAttentionInputs:
    q: torch.Tensor
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    cos: Optional[torch.Tensor] = None
    sin: Optional[torch.Tensor] = None
    rotary_dim: int = 64
    scale: Optional[float] = None


@dataclass(frozen=True)
class LinearAttentionInputs:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    state: torch.Tensor
    decay: float = 1.0


@dataclass(frozen=True)
class AttentionBlockInputs:
    """A full-attention block with its projections: what the decode task graph calls `rmsnorm`, `linear`
    (q | k | v), `attention` and `linear_residual` (mpk_graph.py).  No counterpart in the reference's ops,
    whose decode layer starts from q and the caches.

    qkv_weight [(Hq + 2 Hkv) * D, hidden]: rows of the query heads, then the key heads, then the value
    heads.  out_weight [hidden, Hq * D].  k_cache / v_cache [B, T_max, Hkv, D] hold the first `position`
    tokens; the new token's key and value are written at `position` (in place) and attention runs over
    `position + 1` tokens.  cos / sin [rotary_dim] are those of `position`; they rotate the new query and
    the new key only (the cache keeps rotated keys)."""

    input_norm_weight: torch.Tensor
    qkv_weight: torch.Tensor
    out_weight: torch.Tensor
    k_cache: torch.Tensor
    v_cache: torch.Tensor
    position: int
    query_heads: int
    kv_heads: int
    head_dim: int
    cos: Optional[torch.Tensor] = None
    sin: Optional[torch.Tensor] = None
    rotary_dim: int = 64
    scale: Optional[float] = None


@dataclass(frozen=True)
class DecodeLayerResult:
    hidden: torch.Tensor
    router_indices: Optional[torch.Tensor] = None
    router_weights: Optional[torch.Tensor] = None
    attention_output: Optional[torch.Tensor] = None
    linear_output: Optional[torch.Tensor] = None
    linear_state: Optional[torch.Tensor] = None


_MOE_BACKENDS = ("auto", "persistent", "grouped", "reference")
_DENSE_BACKENDS = ("auto", "torch", "triton", "reference")


def extension_available() -> bool:
    """True when the compiled extension ``mega_kernel_qwen36._C`` could be imported."""
    return _C is not None


def _native(op: str, *tensors: torch.Tensor):
    """The extension module, or a loud failure: this package has no other way to compute."""
    if _C is None:
        raise RuntimeError(
            f"{op}: the sm_100a CUDA extension mega_kernel_qwen36._C is not built or failed to load "
            f"({_IMPORT_ERROR!r}); run build.py. There is no CPU or PyTorch fallback."
        )
    for t in tensors:
        if not t.is_cuda:
            raise RuntimeError(f"{op}: all tensors must be CUDA tensors; this package has no CPU path")
    return _C


def _no_reference(op: str):
    raise RuntimeError(
        f"{op}: backend='reference' names the PyTorch CPU implementation, which is not part of this "
        "package; use any other backend name to run the CUDA kernel"
    )


def moe_decode(
    x: torch.Tensor,
    weights: MoeWeights,
    *,
    eps: float = 1e-6,
    top_k: int = 8,
    add_residual: bool = True,
    backend: str = "auto",
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """RMSNorm -> router top-k (softmax over the k survivors) -> routed + shared SwiGLU experts
    -> residual.  Returns ``(out[B,H], indices[B,K] int64, weights[B,K] float32)``."""
    if backend not in _MOE_BACKENDS:
        raise ValueError("backend must be one of: auto, persistent, grouped, reference")
    if backend == "reference":
        _no_reference("moe_decode")
    tensors = (
        x,
        weights.norm_weight,
        weights.router_weight,
        weights.expert_gate,
        weights.expert_up,
        weights.expert_down,
        weights.shared_gate,
        weights.shared_up,
        weights.shared_down,
    )
    ext = _native("moe_decode", *tensors)
    return ext.moe_decode_persistent(*tensors, float(eps), int(top_k), bool(add_residual))


def dense_ffn_decode(
    x: torch.Tensor,
    weights: DenseFfnWeights,
    *,
    eps: float = 1e-6,
    add_residual: bool = True,
    backend: str = "auto",
) -> torch.Tensor:
    """RMSNorm -> silu(x Wg^T) * (x Wu^T) -> Wd -> residual."""
    if backend not in _DENSE_BACKENDS:
        raise ValueError("backend must be one of: auto, torch, triton, reference")
    if backend == "reference":
        _no_reference("dense_ffn_decode")
    tensors = (x, weights.norm_weight, weights.gate_weight, weights.up_weight, weights.down_weight)
    ext = _native("dense_ffn_decode", *tensors)
    return ext.dense_ffn_decode(*tensors, float(eps), bool(add_residual))


def linear_decode(
    x: torch.Tensor,
    weight: torch.Tensor,
    *,
    norm_weight: Optional[torch.Tensor] = None,
    residual: Optional[torch.Tensor] = None,
    eps: float = 1e-6,
    return_argmax: bool = False,
):
    """Decode-time projection ``weight @ (rms_norm(x) or x) (+ residual)`` for up to eight tokens.

    The `linear` (q/k/v), `linear_residual` (attention output) and `lm_head` tasks of the decode task
    graph (mpk_graph.py), which the reference plans but leaves to the caller.  x [B, K]; weight [N, K];
    norm_weight [K] fuses the RMSNorm (rounded to x.dtype, as reference.py:10-13 does); residual
    [B, N] is added in fp32 before the single rounding.  With ``return_argmax`` also returns int64 [B]:
    arg-max of each stored output row, lowest index among equals."""
    ext = _native("linear_decode", x, weight)
    out, best = ext.linear_decode(x, weight, norm_weight, residual, float(eps), bool(return_argmax))
    return (out, best) if return_argmax else out


def apply_partial_rope(
    q: torch.Tensor,
    k: torch.Tensor,
    cos: Optional[torch.Tensor],
    sin: Optional[torch.Tensor],
    rotary_dim: int,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotate-half rotary embedding on the first ``rotary_dim`` channels of q and k (the whole
    cache), in fp32, as the reference applies it before attention (reference.py:91-114,
    ops.py:368).  Identity when cos/sin are not given, which is the default."""
    if cos is None or sin is None or rotary_dim <= 0:
        return q, k
    half = rotary_dim // 2

    def rotate(t: torch.Tensor) -> torch.Tensor:
        c = cos.to(device=t.device, dtype=torch.float32)
        s = sin.to(device=t.device, dtype=torch.float32)
        lead = t[..., :rotary_dim].float()
        while c.ndim < lead.ndim:
            c, s = c.unsqueeze(0), s.unsqueeze(0)
        turned = torch.cat((-lead[..., half:], lead[..., :half]), dim=-1)
        return torch.cat(((lead * c + turned * s).to(t.dtype), t[..., rotary_dim:]), dim=-1)

    return rotate(q), rotate(k)


def full_attention_decode(inputs: FullAttentionInputs) -> torch.Tensor:
    """One-token GQA attention over the whole KV cache.  q [B,Hq,D]; caches [B,T,Hkv,D]."""
    ext = _native("full_attention_decode", inputs.q, inputs.k_cache, inputs.v_cache)
    q, k_cache = apply_partial_rope(inputs.q, inputs.k_cache, inputs.cos, inputs.sin, inputs.rotary_dim)
    scale = inputs.scale
    if scale is None:
        scale = 1.0 / math.sqrt(q.shape[-1])
    return ext.full_attention_decode(q.contiguous(), k_cache.contiguous(), inputs.v_cache.contiguous(), float(scale))


def attention_block_decode(hidden: torch.Tensor, block: AttentionBlockInputs, *, eps: float = 1e-6) -> Tuple[torch.Tensor, torch.Tensor]:
    """hidden [B, H] -> (hidden + out_proj(attention(q, cache)), attention output [B, Hq, D]).

    Three launches: the fused RMSNorm + q|k|v projection, the attention kernel over the cache including
    the new token, and the output projection with the residual added before the single rounding."""
    hq, hkv, d = block.query_heads, block.kv_heads, block.head_dim
    b = hidden.shape[0]
    if block.qkv_weight.shape[0] != (hq + 2 * hkv) * d:
        raise ValueError("qkv_weight must have (query_heads + 2 * kv_heads) * head_dim rows")
    if not 0 <= block.position < block.k_cache.shape[1]:
        raise ValueError("position must lie inside the cache")
    qkv = linear_decode(hidden, block.qkv_weight, norm_weight=block.input_norm_weight, eps=eps)
    q = qkv[:, : hq * d].reshape(b, hq, d)
    k_new = qkv[:, hq * d : (hq + hkv) * d].reshape(b, 1, hkv, d)
    v_new = qkv[:, (hq + hkv) * d :].reshape(b, 1, hkv, d)
    q, k_new = apply_partial_rope(q, k_new, block.cos, block.sin, block.rotary_dim)
    t = block.position + 1
    block.k_cache[:, block.position : t] = k_new
    block.v_cache[:, block.position : t] = v_new
    k_used, v_used = block.k_cache[:, :t], block.v_cache[:, :t]
    if not k_used.is_contiguous():  # batch > 1 with a cache longer than the context: the kernel wants dense [B, T, Hkv, D]
        k_used, v_used = k_used.contiguous(), v_used.contiguous()
    attn = full_attention_decode(FullAttentionInputs(q=q.contiguous(), k_cache=k_used, v_cache=v_used, scale=block.scale))
    out = linear_decode(attn.reshape(b, hq * d), block.out_weight, residual=hidden)
    return out, attn


def linear_attention_decode(inputs: LinearAttentionInputs) -> Tuple[torch.Tensor, torch.Tensor]:
    """``S' = decay*S + k (x) v``, ``out = q^T S'``.  Returns ``(out, new_state)``; the input
    state is not modified."""
    ext = _native("linear_attention_decode", inputs.q, inputs.k, inputs.v, inputs.state)
    return ext.linear_attention_decode(
        inputs.q.contiguous(),
        inputs.k.contiguous(),
        inputs.v.contiguous(),
        inputs.state.contiguous(),
        float(inputs.decay),
    )


def linear_attention_decode_gated(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    state: torch.Tensor,
    *,
    decay: float = 1.0,
    decay_per_head: Optional[torch.Tensor] = None,
    beta_per_head: Optional[torch.Tensor] = None,
    inplace: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Extension of ``linear_attention_decode``: per-(batch, value head) decay and value scale
    (``S' = decay[b,h]*S + k (x) (beta[b,h]*v)``), fewer key heads than value heads (key head
    ``h // (Hv/Hk)`` serves value head ``h``) and an optional in-place state update.  With the
    defaults it is the same computation as ``linear_attention_decode``."""
    ext = _native("linear_attention_decode", q, k, v, state)
    return ext.linear_attention_decode_ex(
        q.contiguous(), k.contiguous(), v.contiguous(), state if inplace else state.contiguous(),
        float(decay), decay_per_head, beta_per_head, bool(inplace),
    )


def linear_attention_decode_steps(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    state: torch.Tensor,
    *,
    decay: float = 1.0,
    decay_per_step: Optional[torch.Tensor] = None,
    beta_per_step: Optional[torch.Tensor] = None,
    inplace: bool = False,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Several consecutive steps of the recurrence in one launch with the fp32 state resident on
    chip: ``q, k`` are ``[steps, B, Hk, Dk]``, ``v`` is ``[steps, B, Hv, Dv]``; returns
    ``(out[steps, B, Hv, Dv], final_state)``.  Bit-identical to ``steps`` calls of
    ``linear_attention_decode`` / ``linear_attention_decode_gated`` (the gates are then
    ``[steps, B, Hv]``), but the state crosses HBM twice per call instead of twice per step."""
    ext = _native("linear_attention_decode_steps", q, k, v, state)
    return ext.linear_attention_decode_steps(
        q.contiguous(), k.contiguous(), v.contiguous(), state if inplace else state.contiguous(),
        float(decay), decay_per_step, beta_per_step, bool(inplace),
    )


def decode_layer(
    layer_idx: int,
    hidden: torch.Tensor,
    moe: Optional[MoeWeights] = None,
    *,
    dense_ffn: Optional[DenseFfnWeights] = None,
    full_attention: Optional[FullAttentionInputs] = None,
    linear_attention: Optional[LinearAttentionInputs] = None,
    layer_type: Optional[str] = None,
    eps: float = 1e-6,
    top_k: int = 8,
    attention_block: Optional[AttentionBlockInputs] = None,
) -> DecodeLayerResult:
    """Token mixer (full attention every fourth layer, the linear recurrence otherwise), residual
    add, then the dense or MoE feed-forward with its own residual.  The mixer output is reshaped to
    the hidden shape, so ``heads * head_dim`` must equal the hidden size (ops.py:722-729) - unless
    ``attention_block`` supplies the block's own projections (an extension: any head geometry)."""
    kind = layer_type or qwen36_layer_type(layer_idx)
    attention_output = linear_output = linear_state = None
    if kind == "full_attention" and attention_block is not None:
        stream, attention_output = attention_block_decode(hidden, attention_block, eps=eps)
    elif kind == "full_attention":
        if full_attention is None:
            raise ValueError("full_attention inputs are required for full_attention layers")
        attention_output = full_attention_decode(full_attention).reshape_as(hidden)
        stream = hidden + attention_output
    elif kind == "linear_attention":
        if linear_attention is None:
            raise ValueError("linear_attention inputs are required for linear_attention layers")
        linear_output, linear_state = linear_attention_decode(linear_attention)
        linear_output = linear_output.reshape_as(hidden)
        stream = hidden + linear_output
    else:
        raise ValueError(f"unsupported layer_type: {kind}")

    router_indices = router_weights = None
    if dense_ffn is not None:
        out = dense_ffn_decode(stream, dense_ffn, eps=eps, add_residual=True)
    else:
        if moe is None:
            raise ValueError("either moe or dense_ffn weights are required")
        out, router_indices, router_weights = moe_decode(stream, moe, eps=eps, top_k=top_k, add_residual=True)
    return DecodeLayerResult(
        hidden=out,
        router_indices=router_indices,
        router_weights=router_weights,
        attention_output=attention_output,
        linear_output=linear_output,
        linear_state=linear_state,
    )
