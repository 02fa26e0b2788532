"""Sharding of the decode layer over the GPUs of one NVLink/NVSwitch box (one process per GPU).

The reference is single-GPU only (README.md:6-7; no collective anywhere in its tree), so there
is nothing to mirror here.  Three partitions follow the structure of the ops:

  * MoE - expert parallel.  Rank r holds experts [r*E/N, (r+1)*E/N) and 1/N of the shared
    expert's intermediate rows.  Every rank runs the router on the replicated token (the kernel
    is deterministic, so all ranks select the same experts without exchanging indices), computes
    the contribution of its local experts as an fp32 partial [B, H], and one all-reduce sums the
    partials; the residual is added once, after the reduction.
  * dense FFN - tensor parallel.  Gate/up are split by rows, down by columns (stored densely per
    rank); the same single all-reduce of an fp32 [B, H] partial.
  * attention - KV-head parallel.  Rank r owns KV heads [r*Hkv/N, ...) and their query heads; no
    exchange is needed, an all-gather only if every rank wants the full output.

The collective is NCCL through ``torch.distributed`` (gloo on CPU for tests).  The partial sums
leave the kernels in fp32 and are reduced in fp32, so the result does not depend on the number
of ranks beyond fp32 reassociation.
"""

from __future__ import annotations

from dataclasses import dataclass
from typing import Optional, Tuple

import torch
import torch.distributed as dist

from .ops import DenseFfnWeights, FullAttentionInputs, MoeWeights, _native


def _span(total: int, rank: int, world: int) -> Tuple[int, int]:
    """Contiguous share [begin, end) of `total` items for `rank`; `total` must divide evenly so
    that every rank streams the same number of bytes."""
    if world <= 0 or not 0 <= rank < world:
        raise ValueError(f"invalid rank {rank} for world size {world}")
    if total % world != 0:
        raise ValueError(f"{total} items cannot be split evenly over {world} ranks")
    per = total // world
    return rank * per, (rank + 1) * per


@dataclass(frozen=True)
class MoeShard:
    weights: MoeWeights      # router and norm replicated; expert slabs and shared slices local
    expert_base: int         # global id of the first local expert
    rank: int
    world: int


def shard_moe_weights(weights: MoeWeights, rank: int, world: int) -> MoeShard:
    """Expert-parallel slice of a full set of MoE weights (works on any device)."""
    experts = weights.router_weight.shape[0]
    e0, e1 = _span(experts, rank, world)
    s0, s1 = _span(weights.shared_gate.shape[0], rank, world)
    local = MoeWeights(
        norm_weight=weights.norm_weight,
        router_weight=weights.router_weight,
        expert_gate=weights.expert_gate[e0:e1].contiguous(),
        expert_up=weights.expert_up[e0:e1].contiguous(),
        expert_down=weights.expert_down[e0:e1].contiguous(),
        shared_gate=weights.shared_gate[s0:s1].contiguous(),
        shared_up=weights.shared_up[s0:s1].contiguous(),
        shared_down=weights.shared_down[:, s0:s1].contiguous(),
    )
    return MoeShard(local, e0, rank, world)


def shard_dense_weights(weights: DenseFfnWeights, rank: int, world: int) -> DenseFfnWeights:
    """Tensor-parallel slice: rows of gate/up, the matching columns of down stored densely."""
    i0, i1 = _span(weights.gate_weight.shape[0], rank, world)
    return DenseFfnWeights(
        norm_weight=weights.norm_weight,
        gate_weight=weights.gate_weight[i0:i1].contiguous(),
        up_weight=weights.up_weight[i0:i1].contiguous(),
        down_weight=weights.down_weight[:, i0:i1].contiguous(),
    )


def shard_attention_inputs(inputs: FullAttentionInputs, rank: int, world: int) -> FullAttentionInputs:
    """KV-head-parallel slice: the rank's KV heads and the query heads that read them."""
    kv_heads = inputs.k_cache.shape[2]
    group = inputs.q.shape[1] // kv_heads
    k0, k1 = _span(kv_heads, rank, world)
    return FullAttentionInputs(
        q=inputs.q[:, k0 * group:k1 * group].contiguous(),
        k_cache=inputs.k_cache[:, :, k0:k1].contiguous(),
        v_cache=inputs.v_cache[:, :, k0:k1].contiguous(),
        cos=inputs.cos, sin=inputs.sin, rotary_dim=inputs.rotary_dim,
        scale=inputs.scale if inputs.scale is not None else 1.0 / float(inputs.q.shape[-1]) ** 0.5,
    )


def combine_partials(partial: torch.Tensor, x: torch.Tensor, *, add_residual: bool = True,
                     group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Sums the ranks' fp32 partials [B, H] in place (all-reduce), adds the residual once and
    rounds to the activation dtype.  Works for NCCL (CUDA tensors) and gloo (CPU tensors)."""
    if partial.dtype != torch.float32:
        raise ValueError("partials must be float32")
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(partial, op=dist.ReduceOp.SUM, group=group)
    if add_residual:
        partial = partial + x.float()
    return partial.to(x.dtype)


def moe_decode_ep(x: torch.Tensor, shard: MoeShard, *, eps: float = 1e-6, top_k: int = 8, add_residual: bool = True,
                  group: Optional[dist.ProcessGroup] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Expert-parallel ``moe_decode``: x is replicated on every rank; returns the full output on
    every rank plus the (identical on all ranks) routing."""
    w = shard.weights
    tensors = (x, w.norm_weight, w.router_weight, w.expert_gate, w.expert_up, w.expert_down,
               w.shared_gate, w.shared_up, w.shared_down)
    ext = _native("moe_decode_ep", *tensors)
    partial, idx, rw = ext.moe_decode_partial(*tensors, float(eps), int(top_k), int(shard.expert_base))
    return combine_partials(partial, x, add_residual=add_residual, group=group), idx, rw


def dense_ffn_decode_tp(x: torch.Tensor, local: DenseFfnWeights, *, eps: float = 1e-6, add_residual: bool = True,
                        group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """Tensor-parallel ``dense_ffn_decode``: one all-reduce of the fp32 partial."""
    tensors = (x, local.norm_weight, local.gate_weight, local.up_weight, local.down_weight)
    ext = _native("dense_ffn_decode_tp", *tensors)
    partial = ext.dense_ffn_decode_partial(*tensors, float(eps))
    return combine_partials(partial, x, add_residual=add_residual, group=group)


def full_attention_decode_kvp(local: FullAttentionInputs, *, gather: bool = False,
                              group: Optional[dist.ProcessGroup] = None) -> torch.Tensor:
    """KV-head-parallel attention on this rank's head slice.  With ``gather`` the slices of all
    ranks are concatenated along the head axis on every rank."""
    from .ops import full_attention_decode

    out = full_attention_decode(local)
    if gather and dist.is_initialized() and dist.get_world_size(group) > 1:
        parts = [torch.empty_like(out) for _ in range(dist.get_world_size(group))]
        dist.all_gather(parts, out, group=group)
        out = torch.cat(parts, dim=1)
    return out
