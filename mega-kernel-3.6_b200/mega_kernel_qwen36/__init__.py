"""B200-native Qwen3.6 single-token decode layer.

Same import surface as the decode part of the reference package ``mega_kernel_qwen36``
(``__init__.py:1-89`` there): configuration dataclasses, the MPK-style planner and the five
decode operators.  The vision-encoder names of the reference are not provided.
"""

from .config import (
    Qwen36TextConfig,
    qwen36_27b_config,
    qwen36_35b_a3b_config,
    qwen36_layer_type,
)
from .mpk_graph import (
    CompiledPlan,
    EventSpec,
    KernelLaunch,
    KernelPhase,
    LaunchStep,
    TaskGraph,
    TaskSpec,
    TensorSpec,
    WorkerConfig,
    build_batch_specialized_plans,
    build_qwen36_decode_tgraph,
)
from .ops import (
    AttentionBlockInputs,
    DecodeLayerResult,
    DenseFfnWeights,
    FullAttentionInputs,
    LinearAttentionInputs,
    MoeWeights,
    apply_partial_rope,
    attention_block_decode,
    decode_layer,
    dense_ffn_decode,
    linear_decode,
    extension_available,
    full_attention_decode,
    linear_attention_decode,
    linear_attention_decode_gated,
    linear_attention_decode_steps,
    moe_decode,
)

__all__ = [
    "AttentionBlockInputs",
    "attention_block_decode",
    "CompiledPlan",
    "DecodeLayerResult",
    "DenseFfnWeights",
    "EventSpec",
    "FullAttentionInputs",
    "KernelLaunch",
    "KernelPhase",
    "LaunchStep",
    "LinearAttentionInputs",
    "MoeWeights",
    "Qwen36TextConfig",
    "TaskGraph",
    "TaskSpec",
    "TensorSpec",
    "WorkerConfig",
    "apply_partial_rope",
    "build_batch_specialized_plans",
    "build_qwen36_decode_tgraph",
    "decode_layer",
    "dense_ffn_decode",
    "linear_decode",
    "extension_available",
    "full_attention_decode",
    "linear_attention_decode",
    "linear_attention_decode_gated",
    "linear_attention_decode_steps",
    "moe_decode",
    "qwen36_27b_config",
    "qwen36_35b_a3b_config",
    "qwen36_layer_type",
]
