"""One rank of the multi-GPU parity check (launched by tests/test_multi_gpu.py through torchrun).

Every rank builds the same seeded full weights on the host, keeps its shard on its GPU, and runs
the expert-parallel MoE / tensor-parallel dense FFN with the cross-GPU sum fused into the kernel
(`PeerExchange`), and the KV-head-parallel attention where the head count divides by the world size.  Checked on every rank: the result against the CPU oracle on the full weights
(the tolerances of tests/parity.py), routing bit-exact, the NCCL all-reduce variant within the
same tolerance, several steps in a row (both halves of the double-buffered exchange), and - on
rank 0 - that all ranks hold bit-identical outputs.
"""

import os
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
for p in (str(ROOT), str(ROOT / "mega-kernel-3.6_b200"), str(ROOT / "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

import parity  # noqa: E402


def main() -> int:
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import parallel, synthetic as syn
    from oracle import decode_oracle as oracle

    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    # every rank draws the full weights and runs the CPU oracle on them: share the host cores instead of
    # letting `world` processes start one thread per core each
    torch.set_num_threads(max(1, (os.cpu_count() or 8) // world))
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", rank)))
    torch.cuda.set_device(device)
    dist.init_process_group("nccl", device_id=device)
    failures = []

    def check(fn, *args) -> None:
        # record and carry on: every rank must keep making the same sequence of collective calls
        try:
            fn(*args)
        except AssertionError as exc:
            failures.append(f"rank {rank}: {exc}")

    def same_on_all_ranks(t: torch.Tensor, what: str) -> None:
        parts = [torch.empty_like(t) for _ in range(world)]
        dist.all_gather(parts, t.contiguous())
        for q in range(1, world):
            if not torch.equal(parts[0], parts[q]):
                failures.append(f"{what}: rank {q} differs from rank 0")

    # Each case runs the all-reduce variant first: a local launch of the same kernels, so that module
    # loading on one rank does not eat into the bounded waits of its peers.
    exchange = None
    try:
        # ---------------- MoE, expert parallel ----------------
        moe_cases = [
            ("moe_small_bf16", syn.MOE_SMALL, 3, torch.bfloat16, 4),
            ("moe_small_f32", syn.MOE_SMALL, 2, torch.float32, 4),
            ("moe_35b_b1", syn.MOE_35B_A3B, 1, torch.bfloat16, 8),
            ("moe_35b_b2", syn.MOE_35B_A3B, 2, torch.bfloat16, 8),
            ("moe_35b_b8", syn.MOE_35B_A3B, 8, torch.bfloat16, 8),
        ]
        for name, shape, batch, dtype, top_k in moe_cases:
            host = syn.moe_weights(shape, seed=3, dtype=dtype)
            full = mk.MoeWeights(*[host[f] for f in syn.MOE_WEIGHT_FIELDS])
            base = parallel.shard_moe_weights(full, rank, world)
            shard = parallel.MoeShard(mk.MoeWeights(*[getattr(base.weights, f).to(device) for f in syn.MOE_WEIGHT_FIELDS]),
                                      base.expert_base, rank, world)
            xs = [syn.hidden_states(batch, shape.hidden, seed=40 + i, dtype=dtype) for i in range(3)]
            ref = [oracle.moe_decode(x, *[host[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=top_k) for x in xs]
            # all-reduce variant (also warms the kernels up locally before any peer wait)
            for x, (ro, ri, rw) in zip(xs, ref):
                out, idx, w = parallel.moe_decode_ep(x.to(device), shard, top_k=top_k)
                check(parity.assert_output_parity, out.cpu(), ro, f"{name} nccl")
                check(parity.assert_indices_exact, idx.cpu(), ri)
            torch.cuda.synchronize()
            dist.barrier()
            if exchange is None:
                exchange = parallel.PeerExchange(device)
            for step in range(6):  # both parities of the exchange, three times
                x, (ro, ri, rw) = xs[step % 3], ref[step % 3]
                out, idx, w = parallel.moe_decode_ep(x.to(device), shard, top_k=top_k, exchange=exchange)
                torch.cuda.synchronize()
                status = mk.ops._C.workspace_status(out)
                if status != 0:
                    failures.append(f"{name} step {step}: device status {status}")
                check(parity.assert_output_parity, out.cpu(), ro, f"{name} fused step {step}")
                check(parity.assert_indices_exact, idx.cpu(), ri)
                if not torch.allclose(w.cpu(), rw, rtol=1e-5, atol=1e-6):
                    failures.append(f"{name} step {step}: route weights differ")
                same_on_all_ranks(out, f"{name} step {step}")
            del shard, host, full, base
            torch.cuda.empty_cache()

        # ---------------- dense FFN, tensor parallel ----------------
        dense_cases = [
            ("dense_mid_bf16", syn.DenseShape(256, 704), 3, torch.bfloat16),
            ("dense_27b_b1", syn.DENSE_27B, 1, torch.bfloat16),
        ]
        for name, shape, batch, dtype in dense_cases:
            host = syn.dense_weights(shape, seed=5, dtype=dtype)
            full = mk.DenseFfnWeights(*[host[f] for f in syn.DENSE_WEIGHT_FIELDS])
            cut = parallel.shard_dense_weights(full, rank, world)
            local = mk.DenseFfnWeights(*[getattr(cut, f).to(device) for f in syn.DENSE_WEIGHT_FIELDS])
            x = syn.hidden_states(batch, shape.hidden, seed=9, dtype=dtype)
            ro = oracle.dense_ffn_decode(x, *[host[f] for f in syn.DENSE_WEIGHT_FIELDS])
            out = parallel.dense_ffn_decode_tp(x.to(device), local)
            check(parity.assert_output_parity, out.cpu(), ro, f"{name} nccl")
            torch.cuda.synchronize()
            dist.barrier()
            for step in range(3):
                out = parallel.dense_ffn_decode_tp(x.to(device), local, exchange=exchange)
                torch.cuda.synchronize()
                status = mk.ops._C.workspace_status(out)
                if status != 0:
                    failures.append(f"{name} step {step}: device status {status}")
                check(parity.assert_output_parity, out.cpu(), ro, f"{name} fused step {step}")
                same_on_all_ranks(out, f"{name} step {step}")
            if name == "dense_mid_bf16":
                # the way back after a failed step: clear every rank's exchange buffer (the counters stand at an odd
                # step here), then the same call must give the same bits again
                before = out.clone()
                exchange.reset()
                for step in range(2):
                    again = parallel.dense_ffn_decode_tp(x.to(device), local, exchange=exchange)
                    torch.cuda.synchronize()
                    if not torch.equal(again, before):
                        failures.append(f"{name}: step {step} after the exchange reset differs")
                if mk.ops._C.workspace_status(again) != 0:
                    failures.append(f"{name}: device status set after the exchange reset")
            del local, host, full, cut
            torch.cuda.empty_cache()
        # ---------------- attention, KV-head parallel (no exchange; only where the head count allows) ----------------
        for name, heads, kv_heads, dim, seq in (("attn_35b_t2048", 16, 2, 256, 2048), ("attn_27b_t1000", 24, 4, 256, 1000)):
            if kv_heads % world != 0:
                continue
            t = syn.attention_tensors(1, heads, kv_heads, dim, seq, seed=11)
            scale = 1.0 / float(dim) ** 0.5
            full = mk.FullAttentionInputs(q=t["q"], k_cache=t["k_cache"], v_cache=t["v_cache"], scale=scale)
            cut = parallel.shard_attention_inputs(full, rank, world)
            mine = mk.FullAttentionInputs(q=cut.q.to(device), k_cache=cut.k_cache.to(device), v_cache=cut.v_cache.to(device), scale=cut.scale)
            out = parallel.full_attention_decode_kvp(mine, gather=True)
            ro = oracle.full_attention_decode(t["q"], t["k_cache"], t["v_cache"], scale=scale)
            check(parity.assert_output_parity, out.cpu(), ro, f"{name} kv-head parallel")
            same_on_all_ranks(out, name)
    except AssertionError as exc:  # keep the ranks in step: report, do not leave peers waiting
        failures.append(f"rank {rank}: {exc}")
    torch.cuda.synchronize()
    flag = torch.tensor([len(failures)], device=device)
    dist.all_reduce(flag)
    dist.barrier()
    if exchange is not None:
        exchange.close()
    dist.destroy_process_group()
    for f in failures:
        print(f"FAIL[{rank}] {f}", flush=True)
    if rank == 0:
        print("MULTI_GPU_OK" if int(flag) == 0 else f"MULTI_GPU_FAILED ({int(flag)} failures)", flush=True)
    return 0 if int(flag) == 0 else 1


if __name__ == "__main__":
    sys.exit(main())
