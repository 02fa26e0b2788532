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

Two ways to sum the partials.  The plain one is an all-reduce through ``torch.distributed``
(NCCL on GPUs, gloo on CPU for tests) followed by the residual add.  The fast one is
``PeerExchange``: the kernels themselves store their partial rows into every rank's exchange
buffer over NVLink, signal, wait (bounded) for the peers' rows and finish the output in the same
launch, so a decode step stays one kernel per GPU (``exchange=`` argument below).  The partial
sums are fp32 and are added in rank order on every rank, so all ranks get bit-identical outputs.
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


class PeerExchange:
    """The ranks' exchange buffers for the fused cross-GPU sum (see csrc/mk36_comm.cuh).

    Collective constructor: every rank of `group` calls it once, with its CUDA device current.
    It allocates this rank's buffer (a plain cudaMalloc: CUDA IPC cannot export a slice of a
    caching allocator's block), swaps IPC handles through the process group and maps the peers'
    buffers.  All ranks must then make the same sequence of ``moe_decode_ep`` /
    ``dense_ffn_decode_tp`` calls with this object.
    """

    def __init__(self, device: torch.device, group: Optional[dist.ProcessGroup] = None):
        from .ops import _C

        if _C is None:
            raise RuntimeError("the sm_100a extension is not built; there is no fallback for the peer exchange")
        self._ext = _C
        self.rank = dist.get_rank(group)
        self.world = dist.get_world_size(group)
        self.device = torch.device(device)
        self._own = 0
        self._peers = {}
        with torch.cuda.device(self.device):
            self._own = int(_C.comm_buffer_alloc())
            handle = bytes(_C.ipc_export(self._own))
            handles = [None] * self.world
            dist.all_gather_object(handles, handle, group=group)
            for q, h in enumerate(handles):
                if q != self.rank:
                    self._peers[q] = int(_C.ipc_open(h))
        self.buffers = [self._own if q == self.rank else self._peers[q] for q in range(self.world)]
        dist.barrier(group=group)  # every buffer is cleared and mapped everywhere before the first step

    def reset(self, group: Optional[dist.ProcessGroup] = None) -> None:
        """Collective: clears every rank's buffer (step counters and slots).  The way back after a step in which a
        rank gave up waiting for a peer, which leaves the ranks' step counters in disagreement; the workspaces
        whose status was set must be re-initialised as well (``workspace_reset`` of the extension)."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            dist.barrier(group=group)  # no rank is still inside a step
            self._ext.comm_buffer_reset(self._own)
            torch.cuda.synchronize()
            dist.barrier(group=group)  # nobody starts the next step against a buffer that is not clear yet

    def close(self) -> None:
        """Unmaps the peers' buffers and frees the own one.  Collective in spirit: no rank may still
        be inside a step that uses this object."""
        with torch.cuda.device(self.device):
            torch.cuda.synchronize()
            for ptr in self._peers.values():
                self._ext.ipc_close(ptr)
            self._peers = {}
            if self._own:
                self._ext.comm_buffer_free(self._own)
                self._own = 0


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
                  group: Optional[dist.ProcessGroup] = None,
                  exchange: Optional[PeerExchange] = None) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Expert-parallel ``moe_decode``: x is replicated on every rank; returns the full output on
    every rank plus the (identical on all ranks) routing.  With ``exchange`` the sum over the
    ranks happens inside the kernel (one launch per step); without it, through an all-reduce."""
    w = shard.weights
    tensors = (x, w.norm_weight, w.router_weight, w.expert_gate, w.expert_up, w.expert_down,
               w.shared_gate, w.shared_up, w.shared_down)
    ext = _native("moe_decode_ep", *tensors)
    if exchange is not None:
        return ext.moe_decode_ep(*tensors, float(eps), int(top_k), bool(add_residual), int(shard.expert_base),
                                 exchange.rank, exchange.world, exchange.buffers)
    partial, idx, rw = ext.moe_decode_partial(*tensors, float(eps), int(top_k), int(shard.expert_base))
    return combine_partials(partial, x, add_residual=add_residual, group=group), idx, rw


def dense_ffn_decode_tp(x: torch.Tensor, local: DenseFfnWeights, *, eps: float = 1e-6, add_residual: bool = True,
                        group: Optional[dist.ProcessGroup] = None, exchange: Optional[PeerExchange] = None) -> torch.Tensor:
    """Tensor-parallel ``dense_ffn_decode``: the fp32 partials are summed inside the kernel
    (``exchange``) or by one all-reduce."""
    tensors = (x, local.norm_weight, local.gate_weight, local.up_weight, local.down_weight)
    ext = _native("dense_ffn_decode_tp", *tensors)
    if exchange is not None:
        return ext.dense_ffn_decode_tp(*tensors, float(eps), bool(add_residual), exchange.rank, exchange.world, exchange.buffers)
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
