"""Sharding logic of the multi-GPU paths on CPU ranks (gloo, world size 2).

The partition functions and the combine step of mega_kernel_qwen36.parallel run unchanged on CPU
tensors; the per-rank kernel is replaced by the CPU oracle evaluated on the rank's shard.  What is
checked: the shards tile the weights exactly, every rank reaches the same routing, and
"sum of the ranks' fp32 partials + residual" equals the unsharded oracle - for the expert-parallel
MoE, the tensor-parallel dense FFN and KV-head-parallel attention.
"""

import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import mega_kernel_qwen36 as mk
from mega_kernel_qwen36 import parallel, synthetic as syn
from oracle import decode_oracle as oracle

WORLD = 2


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _moe_partial_on_cpu(x, shard, top_k, eps=1e-6):
    """What a rank's kernel computes: routing over all experts, contributions of the local experts
    and of the local slice of the shared expert, fp32, no residual."""
    w = shard.weights
    xn = oracle.rms_norm(x, w.norm_weight, eps).float()
    logits = xn @ w.router_weight.float().t()
    best, idx = torch.topk(logits, k=top_k, dim=-1)
    rw = torch.softmax(best, dim=-1)
    acc = torch.zeros(x.shape, dtype=torch.float32)
    n_local = w.expert_gate.shape[0]
    for t in range(x.shape[0]):
        for s in range(top_k):
            e = int(idx[t, s]) - shard.expert_base
            if 0 <= e < n_local:
                act = torch.nn.functional.silu(w.expert_gate[e].float() @ xn[t]) * (w.expert_up[e].float() @ xn[t])
                acc[t] += rw[t, s] * (w.expert_down[e].float() @ act)
    sh = torch.nn.functional.silu(xn @ w.shared_gate.float().t()) * (xn @ w.shared_up.float().t())
    acc += sh @ w.shared_down.float().t()
    return acc, idx, rw


def _dense_partial_on_cpu(x, local, eps=1e-6):
    xn = oracle.rms_norm(x, local.norm_weight, eps).float()
    act = torch.nn.functional.silu(xn @ local.gate_weight.float().t()) * (xn @ local.up_weight.float().t())
    return act @ local.down_weight.float().t()


def _worker(rank: int, port: int, failures):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=WORLD)
    try:
        torch.set_num_threads(2)
        # ---- expert-parallel MoE ----
        t = syn.moe_tensors(syn.MoeShape(128, 16, 4, 64, 32), batch=5, seed=40, dtype=torch.bfloat16, norm_jitter=0.05)
        full = mk.MoeWeights(*[t[f] for f in syn.MOE_WEIGHT_FIELDS])
        shard = parallel.shard_moe_weights(full, rank, WORLD)
        assert shard.expert_base == rank * 8 and shard.weights.expert_gate.shape[0] == 8
        assert shard.weights.shared_down.shape == (128, 16) and shard.weights.shared_gate.shape == (16, 128)
        partial, idx, rw = _moe_partial_on_cpu(t["x"], shard, top_k=4)
        out = parallel.combine_partials(partial, t["x"], add_residual=True)
        ref, ridx, rrw = oracle.moe_decode(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=4)
        assert torch.equal(idx, ridx), "ranks must reach the same routing as the unsharded layer"
        gathered = [torch.empty_like(idx) for _ in range(WORLD)]
        dist.all_gather(gathered, idx)
        assert all(torch.equal(g, idx) for g in gathered)
        assert out.dtype == ref.dtype
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=0)
        assert float((out.float() - ref.float()).norm() / ref.float().norm()) < 1e-2

        # ---- tensor-parallel dense FFN ----
        d = syn.dense_tensors(syn.DenseShape(96, 160), batch=3, seed=41, dtype=torch.bfloat16, norm_jitter=0.05)
        dfull = mk.DenseFfnWeights(*[d[f] for f in syn.DENSE_WEIGHT_FIELDS])
        local = parallel.shard_dense_weights(dfull, rank, WORLD)
        assert local.gate_weight.shape == (80, 96) and local.down_weight.shape == (96, 80) and local.down_weight.is_contiguous()
        out = parallel.combine_partials(_dense_partial_on_cpu(d["x"], local), d["x"], add_residual=True)
        ref = oracle.dense_ffn_decode(d["x"], *[d[f] for f in syn.DENSE_WEIGHT_FIELDS])
        torch.testing.assert_close(out.float(), ref.float(), atol=2e-2, rtol=0)
        no_res = parallel.combine_partials(_dense_partial_on_cpu(d["x"], local), d["x"], add_residual=False)
        ref_no = oracle.dense_ffn_decode(d["x"], *[d[f] for f in syn.DENSE_WEIGHT_FIELDS], add_residual=False)
        torch.testing.assert_close(no_res.float(), ref_no.float(), atol=2e-2, rtol=0)

        # ---- KV-head-parallel attention: head slices are independent ----
        a = syn.attention_tensors(2, 8, 2, 32, 70, seed=42, dtype=torch.bfloat16)
        inputs = mk.FullAttentionInputs(q=a["q"], k_cache=a["k_cache"], v_cache=a["v_cache"])
        mine = parallel.shard_attention_inputs(inputs, rank, WORLD)
        assert mine.q.shape == (2, 4, 32) and mine.k_cache.shape == (2, 70, 1, 32)
        part = oracle.full_attention_decode(mine.q, mine.k_cache, mine.v_cache, scale=mine.scale)
        parts = [torch.empty_like(part) for _ in range(WORLD)]
        dist.all_gather(parts, part)
        ref = oracle.full_attention_decode(a["q"], a["k_cache"], a["v_cache"])
        assert torch.equal(torch.cat(parts, dim=1), ref)

        # ---- argument errors ----
        try:
            parallel.shard_moe_weights(full, rank, 3)
            failures.put(f"rank {rank}: uneven split accepted")
        except ValueError:
            pass
        try:
            parallel.combine_partials(partial.half(), t["x"])
            failures.put(f"rank {rank}: non-fp32 partial accepted")
        except ValueError:
            pass
    except Exception as exc:  # report to the parent instead of dying silently
        failures.put(f"rank {rank}: {type(exc).__name__}: {exc}")
    finally:
        dist.destroy_process_group()


def test_sharded_paths_on_two_gloo_ranks():
    ctx = mp.get_context("spawn")
    failures = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, port, failures)) for r in range(WORLD)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(timeout=240)
    alive = [p for p in procs if p.is_alive()]
    for p in alive:
        p.kill()
    msgs = []
    while not failures.empty():
        msgs.append(failures.get())
    assert not alive, "a rank did not finish"
    assert all(p.exitcode == 0 for p in procs), f"exit codes {[p.exitcode for p in procs]} {msgs}"
    assert not msgs, "\n".join(msgs)


def test_shard_spans_tile_the_range():
    for total, world in ((256, 8), (17408, 4), (2, 2)):
        spans = [parallel._span(total, r, world) for r in range(world)]
        assert spans[0][0] == 0 and spans[-1][1] == total
        assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
    with pytest.raises(ValueError):
        parallel._span(10, 0, 3)
    with pytest.raises(ValueError):
        parallel._span(8, 2, 2)
