"""Text-path dimensions of the two Qwen3.6 checkpoints the decode layer is sized for.

Same names and values as the reference's ``mega_kernel_qwen36/config.py`` (Qwen36TextConfig at
config.py:6-38, layer pattern at config.py:69-72, the two factories at config.py:75-97); the
vision-encoder configuration is not part of the decode path and is not provided.
"""

from __future__ import annotations

import dataclasses
from typing import Tuple

FULL_ATTENTION = "full_attention"
LINEAR_ATTENTION = "linear_attention"


def qwen36_layer_type(layer_idx: int) -> str:
    """Layers 3, 7, 11, ... (zero-based) use full attention, all others the linear recurrence."""
    return FULL_ATTENTION if (layer_idx + 1) % 4 == 0 else LINEAR_ATTENTION


@dataclasses.dataclass(frozen=True)
class Qwen36TextConfig:
    # defaults describe Qwen/Qwen3.6-35B-A3B
    model_name: str = "Qwen/Qwen3.6-35B-A3B"
    is_moe: bool = True
    hidden_size: int = 2048
    num_hidden_layers: int = 40
    vocab_size: int = 248320
    max_position_embeddings: int = 262144
    rms_norm_eps: float = 1e-6
    # full attention
    num_attention_heads: int = 16
    num_key_value_heads: int = 2
    head_dim: int = 256
    partial_rotary_factor: float = 0.25
    rope_theta: int = 10_000_000
    full_attention_interval: int = 4
    # linear attention
    linear_num_key_heads: int = 16
    linear_num_value_heads: int = 32
    linear_key_head_dim: int = 128
    linear_value_head_dim: int = 128
    linear_conv_kernel_dim: int = 4
    # feed-forward
    intermediate_size: int = 0
    num_experts: int = 256
    num_experts_per_tok: int = 8
    moe_intermediate_size: int = 512
    shared_expert_intermediate_size: int = 512

    @property
    def rotary_dim(self) -> int:
        return int(self.head_dim * self.partial_rotary_factor)

    @property
    def layer_types(self) -> Tuple[str, ...]:
        return tuple(qwen36_layer_type(i) for i in range(self.num_hidden_layers))


def qwen36_35b_a3b_config() -> Qwen36TextConfig:
    """Qwen/Qwen3.6-35B-A3B: 40 layers, hidden 2048, 256 experts, top-8, expert width 512."""
    return Qwen36TextConfig()


def qwen36_27b_config() -> Qwen36TextConfig:
    """Qwen/Qwen3.6-27B: dense, 64 layers, hidden 5120, FFN width 17408, 24 query / 4 KV heads."""
    return dataclasses.replace(
        Qwen36TextConfig(),
        model_name="Qwen/Qwen3.6-27B",
        is_moe=False,
        hidden_size=5120,
        num_hidden_layers=64,
        num_attention_heads=24,
        num_key_value_heads=4,
        linear_num_value_heads=48,
        intermediate_size=17408,
        num_experts=0,
        num_experts_per_tok=0,
        moe_intermediate_size=0,
        shared_expert_intermediate_size=0,
    )
