"""MPK-style task-graph planner for Qwen3.6 decode, retargeted to the B200 persistent kernels.

Same planning API as the reference's ``mega_kernel_qwen36/mpk_graph.py`` (TensorSpec / TaskSpec /
EventSpec / WorkerConfig / LaunchStep / CompiledPlan / TaskGraph at mpk_graph.py:37-292,
``build_batch_specialized_plans`` :298-307, ``build_qwen36_decode_tgraph`` :310-516): a graph of
named tasks over named tensors, dependencies canonicalised into activation events, and a
linearisation that tags each task ahead-of-time ("aot", its CTA partition is fixed when the plan
is built) or just-in-time ("jit", the partition depends on run-time data).

What is new is the second half of a plan: ``CompiledPlan.kernel_schedule`` groups the tasks into
the cooperative launches the sm_100a library really performs - one persistent kernel per FFN, one
per attention, one per recurrence step - with, for each launch, the C entry point, grid and block
size, its phases, how many grid barriers separate them and the bytes it must stream from HBM.
Tasks that the decode-layer library has no kernel for (embedding, q/k/v and output projections,
lm_head, sampling) stay in the graph and are marked ``entry_point=None`` in the schedule.

The planner is pure host Python and never touches a device.
"""

from __future__ import annotations

import json
from dataclasses import dataclass, field, replace
from typing import Any, Callable, Dict, Iterable, List, Mapping, Optional, Sequence, Tuple, Union

from .config import Qwen36TextConfig, qwen36_27b_config

GridDim = Tuple[int, int, int]
Dim = Union[int, str]

B200_SMS = 148

# task kinds whose CTA partition is known when the plan is built
_STATIC_KINDS = frozenset(
    {
        "metadata", "embed", "rmsnorm", "linear", "rmsnorm_linear", "linear_residual",
        "dense_gate_up", "dense_down", "linear_attention", "moe_router", "argmax",
    }
)
# task kinds whose partition depends on run-time data: the cache length for attention, the
# routing decision for the expert contraction
_DYNAMIC_KINDS = frozenset({"paged_attention", "split_kv_attention", "moe_grouped_experts"})


def _ceil_div(a: int, b: int) -> int:
    return -(-a // b)


def _batch_ladder(max_batch: int) -> Tuple[int, ...]:
    """1, 2, 4, ... up to and including max_batch."""
    if max_batch < 1:
        raise ValueError("max_batch must be positive")
    sizes: List[int] = []
    b = 1
    while b < max_batch:
        sizes.append(b)
        b *= 2
    sizes.append(max_batch)
    return tuple(sizes)


def _tiled_grid(extent: int, workers: int, tile: int = 64) -> GridDim:
    """CTAs for `extent` outputs in tiles, rounded up to whole waves of `workers`."""
    ctas = max(1, _ceil_div(extent, tile))
    if workers > 0 and ctas > workers:
        ctas = _ceil_div(ctas, workers) * workers
    return (ctas, 1, 1)


@dataclass(frozen=True)
class TensorSpec:
    name: str
    dims: Tuple[Dim, ...]
    dtype: str = "bf16"
    io_category: str = "cuda_tensor"


@dataclass(frozen=True)
class TaskSpec:
    id: str
    kind: str
    inputs: Tuple[str, ...] = ()
    outputs: Tuple[str, ...] = ()
    depends_on: Tuple[str, ...] = ()
    grid_dim: GridDim = (1, 1, 1)
    block_dim: GridDim = (128, 1, 1)
    attrs: Mapping[str, Any] = field(default_factory=dict)
    trigger_event: str = ""
    completion_event: str = ""
    launch_mode: str = "aot"
    worker_hint: Optional[int] = None
    scheduler_hint: Optional[int] = None


@dataclass(frozen=True)
class EventSpec:
    id: str
    prerequisites: Tuple[str, ...] = ()
    dependents: Tuple[str, ...] = ()
    fused_from: Tuple[str, ...] = ()


@dataclass(frozen=True)
class WorkerConfig:
    """SM budget of the persistent runtime.  The default is a B200 (148 SMs); the decode kernels
    themselves run one CTA on every SM and need no scheduler SMs, the split is kept for plans
    that are consumed by an MPK-style runtime."""

    total_sms: int = B200_SMS
    scheduler_sms: int = 4
    scheduler_warps_per_sm: int = 4
    shared_memory_page_kb: int = 32

    @property
    def num_workers(self) -> int:
        return max(1, self.total_sms - self.scheduler_sms)

    @property
    def num_local_schedulers(self) -> int:
        return max(1, self.scheduler_sms * self.scheduler_warps_per_sm)

    @classmethod
    def for_device(cls, total_sms: int, *, scheduler_sms: int = 4) -> "WorkerConfig":
        return cls(total_sms=total_sms, scheduler_sms=min(scheduler_sms, max(1, total_sms - 1)))

    @classmethod
    def current_cuda(cls) -> "WorkerConfig":
        """SM count of the current CUDA device, or the B200 default without one."""
        try:
            import torch

            if torch.cuda.is_available():
                props = torch.cuda.get_device_properties(torch.cuda.current_device())
                return cls.for_device(props.multi_processor_count)
        except Exception:
            pass
        return cls()


@dataclass(frozen=True)
class LaunchStep:
    task_id: str
    event_id: str
    launch_mode: str
    worker: Optional[int]
    scheduler: int


@dataclass(frozen=True)
class KernelPhase:
    name: str
    rows: int            # weight / cache rows streamed in this phase (0 for on-chip phases)
    row_bytes: int
    partition: str       # "static" or "runtime"


@dataclass(frozen=True)
class KernelLaunch:
    """One cooperative launch of the sm_100a library and the plan tasks it fuses."""

    name: str
    entry_point: Optional[str]           # symbol in libmk36.so; None = no kernel in this library
    task_ids: Tuple[str, ...]
    grid: int
    block: int
    grid_barriers: int
    phases: Tuple[KernelPhase, ...] = ()
    hbm_bytes: int = 0                   # distinct bytes that must cross HBM once
    layer: Optional[int] = None
    kernel: Optional[str] = None         # the __global__ function that runs
    launches: int = 1                    # launches of that kernel per decode step (a batch may be split)

    def to_dict(self) -> Dict[str, Any]:
        d = dict(self.__dict__)
        d["phases"] = [dict(p.__dict__) for p in self.phases]
        return d


@dataclass(frozen=True)
class CompiledPlan:
    graph: "TaskGraph"
    worker_config: WorkerConfig
    launch_steps: Tuple[LaunchStep, ...]
    batch_size: int
    kernel_schedule: Tuple[KernelLaunch, ...] = ()

    def to_dict(self) -> Dict[str, Any]:
        data = self.graph.to_dict()
        wc = self.worker_config
        data["worker_config"] = {
            "total_sms": wc.total_sms,
            "num_workers": wc.num_workers,
            "scheduler_sms": wc.scheduler_sms,
            "num_local_schedulers": wc.num_local_schedulers,
            "shared_memory_page_kb": wc.shared_memory_page_kb,
        }
        data["batch_size"] = self.batch_size
        data["launch_steps"] = [dict(step.__dict__) for step in self.launch_steps]
        data["kernel_schedule"] = [k.to_dict() for k in self.kernel_schedule]
        return data

    def to_json(self, *, indent: int = 2) -> str:
        return json.dumps(self.to_dict(), indent=indent, sort_keys=True)

    @property
    def hbm_bytes_per_step(self) -> int:
        return sum(k.hbm_bytes for k in self.kernel_schedule)


@dataclass
class TaskGraph:
    name: str
    tensors: Dict[str, TensorSpec] = field(default_factory=dict)
    tasks: List[TaskSpec] = field(default_factory=list)
    events: Dict[str, EventSpec] = field(default_factory=dict)
    start_event: str = "e_start"
    meta: Dict[str, Any] = field(default_factory=dict)

    # ---- construction ----
    def add_tensor(self, name: str, dims: Sequence[Dim], *, dtype: str = "bf16",
                   io_category: str = "cuda_tensor") -> TensorSpec:
        spec = TensorSpec(name, tuple(dims), dtype, io_category)
        self.tensors[name] = spec
        return spec

    def add_task(self, task_id: str, kind: str, *, inputs: Iterable[str] = (), outputs: Iterable[str] = (),
                 depends_on: Iterable[str] = (), grid_dim: GridDim = (1, 1, 1), block_dim: GridDim = (128, 1, 1),
                 attrs: Optional[Mapping[str, Any]] = None) -> TaskSpec:
        if task_id in {t.id for t in self.tasks}:
            raise ValueError(f"duplicate task id: {task_id}")
        task = TaskSpec(task_id, kind, tuple(inputs), tuple(outputs), tuple(depends_on), grid_dim, block_dim,
                        dict(attrs or {}))
        self.tasks.append(task)
        return task

    # ---- events ----
    def normalize(self) -> "TaskGraph":
        """Give every distinct dependency set one activation event; tasks with the same
        prerequisites share it."""
        event_of: Dict[Tuple[str, ...], str] = {(): self.start_event}
        waiting: Dict[str, List[str]] = {self.start_event: []}
        rewritten: List[TaskSpec] = []
        for task in self.tasks:
            deps = tuple(dict.fromkeys(task.depends_on))
            if deps not in event_of:
                event_of[deps] = f"e_{len(event_of)}"
            ev = event_of[deps]
            waiting.setdefault(ev, []).append(task.id)
            rewritten.append(replace(task, depends_on=deps, trigger_event=ev, completion_event=f"e_done_{task.id}"))
        self.events = {
            ev: EventSpec(
                id=ev,
                prerequisites=deps,
                dependents=tuple(waiting.get(ev, ())),
                fused_from=tuple(f"e_after_{d}" for d in deps) if len(deps) > 1 else (),
            )
            for deps, ev in event_of.items()
        }
        self.tasks = rewritten
        return self

    def event_fusion(self) -> "TaskGraph":
        return self.normalize()

    def topological_tasks(self) -> Tuple[TaskSpec, ...]:
        """Kahn's algorithm; ties are broken by task id so the order is reproducible."""
        by_id = {t.id: t for t in self.tasks}
        missing = {d for t in self.tasks for d in t.depends_on if d not in by_id}
        remaining = {t.id: {d for d in t.depends_on} for t in self.tasks}
        users: Dict[str, List[str]] = {}
        for t in self.tasks:
            for d in t.depends_on:
                users.setdefault(d, []).append(t.id)
        ready = sorted(tid for tid, deps in remaining.items() if not deps)
        order: List[TaskSpec] = []
        while ready:
            tid = ready.pop(0)
            order.append(by_id[tid])
            newly = []
            for user in users.get(tid, ()):
                remaining[user].discard(tid)
                if not remaining[user]:
                    newly.append(user)
            if newly:
                ready = sorted(ready + newly)
        if missing or len(order) != len(self.tasks):
            stuck = sorted(set(by_id) - {t.id for t in order})
            raise ValueError(f"cycle or missing task dependency: {stuck}")
        return tuple(order)

    # ---- planning ----
    def linearize(self, worker_config: Optional[WorkerConfig] = None, *, batch_size: int = 1) -> CompiledPlan:
        wc = worker_config or WorkerConfig.current_cuda()
        self.event_fusion()
        steps: List[LaunchStep] = []
        planned: List[TaskSpec] = []
        for ordinal, task in enumerate(self.topological_tasks()):
            if task.kind in _DYNAMIC_KINDS:
                mode, worker = "jit", None
            elif task.kind in _STATIC_KINDS or len(task.depends_on) == 1:
                mode, worker = "aot", ordinal % wc.num_workers
            else:
                mode, worker = "jit", None
            sched = ordinal % wc.num_local_schedulers
            planned.append(replace(task, launch_mode=mode, worker_hint=worker, scheduler_hint=sched))
            steps.append(LaunchStep(task.id, task.trigger_event or self.start_event, mode, worker, sched))
        # keep the user's insertion order for the stored tasks, with the planning fields filled in
        by_id = {t.id: t for t in planned}
        self.tasks = [by_id[t.id] for t in self.tasks]
        schedule = _kernel_schedule(self, wc, batch_size)
        return CompiledPlan(self, wc, tuple(steps), batch_size, schedule)

    # ---- export ----
    def to_dict(self) -> Dict[str, Any]:
        self.event_fusion()
        return {
            "name": self.name,
            "start_event": self.start_event,
            "tensors": [dict(t.__dict__) for t in self.tensors.values()],
            "events": [dict(e.__dict__) for e in self.events.values()],
            "tasks": [{**t.__dict__, "attrs": dict(t.attrs)} for t in self.tasks],
        }

    def to_json(self, *, indent: int = 2) -> str:
        return json.dumps(self.to_dict(), indent=indent, sort_keys=True)


def build_batch_specialized_plans(builder: Callable[[int], TaskGraph], *, max_batch: int,
                                  worker_config: Optional[WorkerConfig] = None) -> Dict[int, CompiledPlan]:
    """One compiled plan per power-of-two batch size up to ``max_batch`` (and ``max_batch``)."""
    return {b: builder(b).linearize(worker_config=worker_config, batch_size=b) for b in _batch_ladder(max_batch)}


# ---------------------------------------------------------------------------------------------
# Qwen3.6 decode graph
# ---------------------------------------------------------------------------------------------
class _Chain:
    """Appends tasks that each depend on the previous one."""

    def __init__(self, graph: TaskGraph):
        self.graph = graph
        self.last: Optional[str] = None

    def then(self, task_id: str, kind: str, **kw) -> str:
        deps = (self.last,) if self.last else ()
        self.graph.add_task(task_id, kind, depends_on=deps, **kw)
        self.last = task_id
        return task_id


def build_qwen36_decode_tgraph(
    config: Optional[Qwen36TextConfig] = None,
    *,
    batch_size: int = 1,
    num_layers: Optional[int] = None,
    include_metadata: bool = True,
    include_sampling: bool = True,
    worker_config: Optional[WorkerConfig] = None,
) -> TaskGraph:
    """Task graph of one decode step: embed, then per layer
    ``rmsnorm -> (qkv linear -> paged attention -> out-proj + residual | linear-attention recurrence)
    -> rmsnorm -> (router -> grouped experts -> down + residual | gate/up -> down + residual)``,
    then final norm, lm_head and sampling."""
    cfg = config or qwen36_27b_config()
    wc = worker_config or WorkerConfig.current_cuda()
    n_layers = cfg.num_hidden_layers if num_layers is None else min(num_layers, cfg.num_hidden_layers)
    B, H = batch_size, cfg.hidden_size
    g = TaskGraph(name=f"{cfg.model_name}:decode:batch{B}")
    g.meta = {"config": cfg, "layers": n_layers}
    chain = _Chain(g)

    g.add_tensor("tokens", (B, "seq"), dtype="int64")
    g.add_tensor("hidden_0", (B, H))
    if include_metadata:
        g.add_tensor("decode_metadata", (B,), dtype="int32")
        chain.then("continuous_batching_update", "metadata", inputs=("tokens",), outputs=("decode_metadata",),
                   attrs={"paged_attention": True, "select_power_of_two_tgraph": True})
    chain.then("embed", "embed", inputs=("tokens",), outputs=("hidden_0",), attrs={"vocab_size": cfg.vocab_size})

    kinds = cfg.layer_types
    for li in range(n_layers):
        L = f"layer_{li}"
        g.add_tensor(f"{L}_attn_norm_out", (B, H))
        g.add_tensor(f"{L}_attn_residual", (B, H))
        chain.then(f"{L}_attn_norm", "rmsnorm", inputs=(f"hidden_{li}",), outputs=(f"{L}_attn_norm_out",),
                   grid_dim=(B, 1, 1))
        if kinds[li] == "full_attention":
            hq, hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            qkv_dim = (hq + 2 * hkv) * hd
            g.add_tensor(f"{L}_qkv", (B, qkv_dim))
            g.add_tensor(f"{L}_attn_out", (B, hq * hd))
            chain.then(f"{L}_qkv_proj", "linear", inputs=(f"{L}_attn_norm_out",), outputs=(f"{L}_qkv",),
                       grid_dim=_tiled_grid(qkv_dim, wc.num_workers), attrs={"projection": "qkv", "head_dim": hd})
            chain.then(f"{L}_paged_attention", "paged_attention", inputs=(f"{L}_qkv", "decode_metadata"),
                       outputs=(f"{L}_attn_out",), grid_dim=(B, hkv, 1),
                       attrs={"causal": True, "kv_heads": hkv, "q_heads": hq, "layer": li})
            chain.then(f"{L}_attn_out_proj_residual", "linear_residual", inputs=(f"{L}_attn_out", f"hidden_{li}"),
                       outputs=(f"{L}_attn_residual",), grid_dim=_tiled_grid(H, wc.num_workers))
        else:
            chain.then(f"{L}_linear_attention_recurrent", "linear_attention",
                       inputs=(f"{L}_attn_norm_out", f"{L}_linear_state"),
                       outputs=(f"{L}_attn_residual", f"{L}_linear_state_next"),
                       grid_dim=(B, cfg.linear_num_key_heads, 1),
                       attrs={"key_heads": cfg.linear_num_key_heads, "value_heads": cfg.linear_num_value_heads,
                              "conv_kernel": cfg.linear_conv_kernel_dim, "layer": li})

        g.add_tensor(f"{L}_ffn_norm_out", (B, H))
        g.add_tensor(f"hidden_{li + 1}", (B, H))
        chain.then(f"{L}_ffn_norm", "rmsnorm", inputs=(f"{L}_attn_residual",), outputs=(f"{L}_ffn_norm_out",),
                   grid_dim=(B, 1, 1), attrs={"layer": li, "ffn": True})
        if cfg.is_moe:
            K, I = cfg.num_experts_per_tok, cfg.moe_intermediate_size
            g.add_tensor(f"{L}_topk_indices", (B, K), dtype="int64")
            g.add_tensor(f"{L}_topk_weights", (B, K), dtype="float32")
            g.add_tensor(f"{L}_expert_acts", (B, K, I))
            chain.then(f"{L}_moe_router_topk", "moe_router", inputs=(f"{L}_ffn_norm_out",),
                       outputs=(f"{L}_topk_indices", f"{L}_topk_weights"), grid_dim=(B, cfg.num_experts, 1),
                       attrs={"experts": cfg.num_experts, "top_k": K, "layer": li})
            chain.then(f"{L}_moe_grouped_experts", "moe_grouped_experts",
                       inputs=(f"{L}_ffn_norm_out", f"{L}_topk_indices", f"{L}_topk_weights"),
                       outputs=(f"{L}_expert_acts",), grid_dim=(B * K, 1, 1),
                       attrs={"intermediate": I, "shared_expert": True, "layer": li})
            chain.then(f"{L}_moe_down_residual", "linear_residual", inputs=(f"{L}_expert_acts", f"{L}_attn_residual"),
                       outputs=(f"hidden_{li + 1}",), grid_dim=_tiled_grid(H, wc.num_workers), attrs={"layer": li, "ffn": True})
        else:
            I = cfg.intermediate_size
            g.add_tensor(f"{L}_dense_mid", (B, I))
            chain.then(f"{L}_dense_gate_up", "dense_gate_up", inputs=(f"{L}_ffn_norm_out",), outputs=(f"{L}_dense_mid",),
                       grid_dim=_tiled_grid(2 * I, wc.num_workers), attrs={"activation": "silu_mul", "layer": li})
            chain.then(f"{L}_dense_down_residual", "dense_down", inputs=(f"{L}_dense_mid", f"{L}_attn_residual"),
                       outputs=(f"hidden_{li + 1}",), grid_dim=_tiled_grid(H, wc.num_workers), attrs={"layer": li})

    g.add_tensor("norm_out", (B, H))
    chain.then("final_norm", "rmsnorm", inputs=(f"hidden_{n_layers}",), outputs=("norm_out",), grid_dim=(B, 1, 1))
    if include_sampling:
        g.add_tensor("logits", (B, cfg.vocab_size))
        g.add_tensor("next_tokens", (B, 1), dtype="int64")
        chain.then("lm_head", "linear", inputs=("norm_out",), outputs=("logits",),
                   grid_dim=_tiled_grid(cfg.vocab_size, wc.num_workers, tile=128))
        chain.then("argmax_or_sampler", "argmax", inputs=("logits",), outputs=("next_tokens",),
                   grid_dim=(wc.num_workers, 1, 1))
    return g.event_fusion()


# ---------------------------------------------------------------------------------------------
# B200 kernel schedule
# ---------------------------------------------------------------------------------------------
# Launch geometry of the kernels in csrc/: threads per CTA, grid-wide barriers per launch.  The numbers
# mirror the constants of the .cu files (kStThreads, kRingThreads, kDenseThreads, kMmaAttnThreads,
# kLinThreads, kDsThreads, kAsThreads); tests/test_host_api.py reads those files and fails when the two drift apart.
KERNEL_GEOMETRY = {
    "moe_decode_stream_kernel": {"block": 416, "grid_barriers": 1, "max_tokens": 1},
    "moe_decode_batch_kernel": {"block": 416, "grid_barriers": 1, "max_tokens": 8},
    "moe_decode_ring_kernel": {"block": 416, "grid_barriers": 2, "max_tokens": 8},
    "dense_ffn_mma_kernel": {"block": 512, "grid_barriers": 1, "max_tokens": 8},
    "attention_decode_stream_kernel": {"block": 288, "grid_barriers": 1},
    "dense_ffn_stream_kernel": {"block": 416, "grid_barriers": 1, "max_tokens": 1},
    "linear_attention_kernel": {"block": 256, "grid_barriers": 0},
    "linear_decode_kernel": {"block": 288, "grid_barriers": 0, "max_tokens": 8},
}
_SMEM_OPTIN = 232448   # bytes of shared memory one CTA may use on sm_100
_RING_STAGE = 32768


def moe_batch_kernel_fits(hidden: int, experts: int, top_k: int, intermediate: int, shared_intermediate: int, sms: int = 148) -> bool:
    """Shape conditions of the launcher in csrc/moe_decode_batch.cu for launches of eight tokens."""
    hr_max = -(-hidden // sms)
    return (hidden % 256 == 0 and sms <= hidden <= 8 * 384 and intermediate % 32 == 0 and shared_intermediate % 32 == 0
            and 0 < intermediate <= 512 and shared_intermediate <= 512 and 0 < top_k <= 8 and experts <= 256
            and hr_max <= 16 and hr_max * intermediate * 2 <= _RING_STAGE and (-(-experts // sms) + 1) * 8 <= 24)


def moe_ring_tokens_per_launch(hidden: int, top_k: int, intermediate: int, shared_intermediate: int, sms: int = 148) -> int:
    """Tokens the MoE ring kernel serves in one launch: the largest power of two <= 8 whose per-pair
    activations (fp32, or bf16 high + low halves) leave room for three 32 KB ring stages beside them -
    the same fit loop as the launcher in csrc/moe_decode_ring.cu."""
    hr_max = -(-hidden // sms)
    tb = 8
    while tb > 1 and tb * top_k > 64:
        tb //= 2
    while tb >= 1:
        pairs = tb * top_k
        used = hr_max * shared_intermediate * 2
        used += max(tb * hidden * 2, (pairs * intermediate + tb * shared_intermediate) * 4)
        used += (pairs + tb) * hr_max * 4 + 3 * 2 * 4 * 128 * 4 + 16 + 64 * (4 + 8 + 4 + 4) + (2 * 6 + 1 + 4) * 8 + 6 * 128
        if (_SMEM_OPTIN - used - 1024) // _RING_STAGE >= 3:
            return tb
        tb //= 2
    return 1


def _kernel_schedule(graph: TaskGraph, wc: WorkerConfig, batch: int, context_len: int = 32768) -> Tuple[KernelLaunch, ...]:
    """Groups the graph's tasks into the launches libmk36 performs.  The byte counts are the
    distinct bytes each launch must read or write in HBM (bf16 weights and cache, fp32 state); for
    the MoE the number of distinct experts is taken at its maximum min(batch * top_k, experts)."""
    cfg = graph.meta.get("config") if graph.meta else None
    if cfg is None:
        return ()
    H, sms = cfg.hidden_size, wc.total_sms
    by_layer: Dict[Optional[int], List[TaskSpec]] = {}
    launches: List[KernelLaunch] = []
    tasks = {t.id: t for t in graph.tasks}

    def other(task: TaskSpec) -> KernelLaunch:
        return KernelLaunch(name=task.id, entry_point=None, task_ids=(task.id,), grid=task.grid_dim[0],
                            block=task.block_dim[0], grid_barriers=0)

    held_norms: Dict[str, TaskSpec] = {}
    held_head: List[TaskSpec] = []

    def projection_launch(name: str, group, n_in: int, n_out: int, norm: bool, residual: bool, argmax: bool) -> KernelLaunch:
        geo = KERNEL_GEOMETRY["linear_decode_kernel"]
        rows = max(1, _RING_STAGE // (n_in * 2))
        chunks = _ceil_div(n_out, rows)
        phases = ((KernelPhase("rmsnorm_to_smem", 0, 0, "static"),) if norm else ()) + (
            KernelPhase("weight_rows" + ("_residual" if residual else "") + ("_argmax" if argmax else ""), n_out, n_in * 2, "static"),)
        nbytes = n_out * n_in * 2 + batch * (n_in + n_out) * 2 + (n_in * 2 if norm else 0) + (batch * n_out * 2 if residual else 0)
        return KernelLaunch(name=name, entry_point="mk36_linear_decode", task_ids=tuple(t.id for t in group), kernel="linear_decode_kernel",
                            launches=_ceil_div(batch, geo["max_tokens"]), grid=min(sms, chunks), block=geo["block"], grid_barriers=0,
                            phases=phases, hbm_bytes=nbytes)

    for task in graph.topological_tasks():
        li = task.attrs.get("layer")
        if task.kind == "paged_attention":
            hq, hkv, hd = cfg.num_attention_heads, cfg.num_key_value_heads, cfg.head_dim
            row = hkv * hd * 2
            launches.append(KernelLaunch(
                name=f"layer_{li}_attention", entry_point="mk36_full_attention_decode", task_ids=(task.id,),
                kernel="attention_decode_stream_kernel", grid=sms, block=KERNEL_GEOMETRY["attention_decode_stream_kernel"]["block"],
                grid_barriers=KERNEL_GEOMETRY["attention_decode_stream_kernel"]["grid_barriers"], layer=li,
                phases=(KernelPhase("split_kv_online_softmax", 2 * batch * context_len, row, "runtime"),
                        KernelPhase("merge_partials", 0, 0, "static")),
                hbm_bytes=batch * (2 * context_len * row + 2 * hq * hd * 2)))
        elif task.kind == "linear_attention":
            hk, hv = cfg.linear_num_key_heads, cfg.linear_num_value_heads
            dk, dv = cfg.linear_key_head_dim, cfg.linear_value_head_dim
            launches.append(KernelLaunch(
                name=f"layer_{li}_linear_attention", entry_point="mk36_linear_attention_decode", task_ids=(task.id,),
                kernel="linear_attention_kernel", grid=batch * hv * _ceil_div(dv, 32),
                block=KERNEL_GEOMETRY["linear_attention_kernel"]["block"], grid_barriers=0, layer=li,
                phases=(KernelPhase("state_update_and_readout", batch * hv * dk, dv * 4 * 2, "static"),),
                hbm_bytes=2 * batch * hv * dk * dv * 4 + batch * (2 * hk * dk + 2 * hv * dv) * 2))
        elif task.kind == "rmsnorm" and (task.id.endswith("_attn_norm") or task.id == "final_norm"):
            layer_no = int(task.id.split("_")[1]) if task.id.startswith("layer_") else None
            if layer_no is not None and cfg.layer_types[layer_no] != "full_attention":
                launches.append(other(task))  # the recurrence's input norm: not one of this library's launches
            else:
                held_norms[task.id] = task  # fused into the projection that consumes it, if one follows
        elif task.kind == "linear" and task.attrs.get("projection") == "qkv":
            # RMSNorm + q | k | v projection: one launch of the projection kernel
            L = task.id[: -len("_qkv_proj")]
            norm = held_norms.pop(f"{L}_attn_norm", None)
            n_out = (cfg.num_attention_heads + 2 * cfg.num_key_value_heads) * cfg.head_dim
            launches.append(projection_launch(f"{L}_qkv_proj", ([norm] if norm else []) + [task], H, n_out, norm is not None, False, False))
        elif task.kind == "linear_residual" and not task.attrs.get("ffn"):
            launches.append(projection_launch(task.id, [task], cfg.num_attention_heads * cfg.head_dim, H, False, True, False))
        elif task.kind == "linear" and task.id == "lm_head":
            held_head.append(task)
        elif task.kind == "argmax" and held_head:
            norm = held_norms.pop("final_norm", None)
            launches.append(projection_launch("lm_head_argmax", ([norm] if norm else []) + held_head + [task], H, cfg.vocab_size,
                                              norm is not None, False, True))
            held_head.clear()
        elif task.kind == "rmsnorm" and task.attrs.get("ffn"):
            by_layer.setdefault(li, []).append(task)  # fused into the FFN launch below
        elif task.kind in ("moe_router", "moe_grouped_experts", "dense_gate_up"):
            by_layer.setdefault(li, []).append(task)
        elif task.kind == "linear_residual" and task.attrs.get("ffn"):
            group = by_layer.pop(li, []) + [task]
            E, K = cfg.num_experts, cfg.num_experts_per_tok
            I, Is = cfg.moe_intermediate_size, cfg.shared_expert_intermediate_size
            distinct = min(batch * K, E)
            # one token: the stream kernel; more: the batch kernel, eight tokens per launch (the ring
            # kernel, which takes as many tokens per launch as fit beside its activations, for shapes it refuses)
            if batch <= KERNEL_GEOMETRY["moe_decode_stream_kernel"]["max_tokens"]:
                kname, n_launches = "moe_decode_stream_kernel", 1
            elif moe_batch_kernel_fits(H, E, K, I, Is, sms):
                kname = "moe_decode_batch_kernel"
                n_launches = _ceil_div(batch, KERNEL_GEOMETRY[kname]["max_tokens"])
            else:
                kname = "moe_decode_ring_kernel"
                n_launches = _ceil_div(batch, moe_ring_tokens_per_launch(H, K, I, Is, sms))
            geo = KERNEL_GEOMETRY[kname]
            launches.append(KernelLaunch(
                name=f"layer_{li}_moe", entry_point="mk36_moe_decode", task_ids=tuple(t.id for t in group),
                kernel=kname, launches=n_launches, grid=sms, block=geo["block"], grid_barriers=geo["grid_barriers"], layer=li,
                phases=(KernelPhase("rmsnorm_to_smem", 0, 0, "static"),
                        KernelPhase("router_logits", E, H * 2, "static"),
                        KernelPhase("shared_gate_up", 2 * Is, H * 2, "static"),
                        KernelPhase("topk_softmax_group", 0, 0, "static"),
                        KernelPhase("routed_gate_up", distinct * 2 * I, H * 2, "runtime"),
                        KernelPhase("down_and_residual", (distinct + 1) * H, I * 2, "runtime")),
                hbm_bytes=distinct * 3 * I * H * 2 + 3 * Is * H * 2 + E * H * 2 + H * 2 + 2 * batch * H * 2 + batch * K * 12))
        elif task.kind == "dense_down":
            group = by_layer.pop(li, []) + [task]
            I = cfg.intermediate_size
            dense_kernel = "dense_ffn_stream_kernel" if batch == 1 else "dense_ffn_mma_kernel"  # one token streams, more use the tensor cores
            launches.append(KernelLaunch(
                name=f"layer_{li}_dense_ffn", entry_point="mk36_dense_ffn_decode", task_ids=tuple(t.id for t in group),
                kernel=dense_kernel, launches=_ceil_div(batch, KERNEL_GEOMETRY[dense_kernel]["max_tokens"]),
                grid=sms, block=KERNEL_GEOMETRY[dense_kernel]["block"],
                grid_barriers=KERNEL_GEOMETRY[dense_kernel]["grid_barriers"], layer=li,
                phases=(KernelPhase("rmsnorm_to_smem", 0, 0, "static"),
                        KernelPhase("gate_up_swiglu", 2 * I, H * 2, "static"),
                        KernelPhase("down_and_residual", H, I * 2, "static")),
                hbm_bytes=3 * I * H * 2 + H * 2 + 2 * batch * H * 2))
        else:
            launches.append(other(task))
    # norms and heads that no projection launch picked up (linear-attention layers, graphs without sampling)
    for task in list(held_norms.values()) + held_head:
        launches.append(other(task))
    assert not by_layer, f"unscheduled FFN tasks: {by_layer}"
    del tasks
    return tuple(launches)
