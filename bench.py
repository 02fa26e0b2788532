"""Decode-step benchmark of the B200 Qwen3.6 decode layer.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--batch B]

Headline workload: one MoE decode step of the Qwen3.6-35B-A3B layer shape (hidden 2048, 256
experts, top-8, expert width 512, one shared expert of width 512), bf16, batch 1, synthetic
seeded weights ~N(0,0.02) and hidden states ~N(0,1).  One "step" is one pass of the layer over
one batch.  The metric is microseconds per decode step (lower is better); the roofline object
reports the achieved HBM bandwidth (algorithmic bytes / step time) against the measured copy peak.

  * `value`      K steps captured in one CUDA graph (inputs resident in HBM), timed with CUDA
                 events; the steps rotate over several full weight sets whose total size
                 exceeds the L2, so every step streams from HBM.  The graph is replayed several
                 times and the median replay is reported.
  * `e2e`        the same step through the public operator `mega_kernel_qwen36.moe_decode` with
                 the hidden state in pinned host memory: host->device copy, kernel, device->host
                 read of the output, captured once as a CUDA graph per weight set (the way a
                 serving loop issues a fixed step); every timed step refills the pinned input,
                 replays and synchronises.
  * `cpu_baseline` / `--impl reference`  the CPU oracle (a port of the reference's reference.py)
                 on the host cores, same workload.
  * `others`     the remaining decode ops at their measured shapes (MoE batch 8, dense FFN,
                 32K-context attention, linear attention), same method, reported for context.

With N > 1 (torchrun, one rank per GPU) the MoE runs expert-parallel: every rank holds 256/N
experts and 1/N of the shared expert, and the kernels sum the ranks' fp32 partial outputs over
peer memory in their epilogue (strong scaling: the total work is fixed).  Outside the timed
region every N > 1 run checks one fused step of each sharded op against the CPU oracle on the
full weights and that all ranks hold bit-identical outputs (`parity` in the line; a failure
makes the run exit non-zero).
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mega-kernel-3.6_b200"))

import torch  # noqa: E402

FALLBACK_HBM_GBS = 6650.0
NOMINAL_HBM_GBS = 8000.0
L2_BYTES = 126 * 1024 * 1024

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel: read from the ncu
# summary under profiles/ (a line "traffic_bytes_per_launch: N"); None where no capture exists.
NCU_SUMMARY = {1: "moe_decode_stream_kernel_35b_b1.md", 8: "moe_decode_batch_kernel_35b_b8.md"}


def ncu_traffic_bytes(batch: int):
    name = NCU_SUMMARY.get(batch)
    path = ROOT / "profiles" / name if name else None
    if path is None or not path.exists():
        return None
    for line in path.read_text().splitlines():
        if line.strip().lower().startswith("traffic_bytes_per_launch:"):
            try:
                return int(float(line.split(":", 1)[1].strip().replace("_", "").replace(",", "")))
            except ValueError:
                return None
    return None


def measured_peak():
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            return float(json.loads(path.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return FALLBACK_HBM_GBS, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.lines = []
        self.thread = None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


# ---------------------------------------------------------------------------------------------
REPLAYS = 11


def time_graph(step_fns, warmup: int, replays: int = REPLAYS):
    """Captures the given step callables (one launch each) in one CUDA graph and times `replays`
    replays, each with its own pair of CUDA events on the capture stream.  Returns the median
    replay's milliseconds for all steps, the graph, the stream and the list of replay times."""
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        for i in range(warmup):
            step_fns[i % len(step_fns)]()
        stream.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            for fn in step_fns:
                fn()
        graph.replay()  # untimed replay: graph upload and first-touch effects
        stream.synchronize()
        times = []
        for _ in range(max(1, replays)):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
            times.append(start.elapsed_time(end))
        return statistics.median(times), graph, stream, times


def hold_load(graph, stream, replays: int):
    """Replays a captured graph `replays` more times (untimed) so that the clock sampler, which
    cannot sample faster than every 100 ms, sees the same load as the few-millisecond timed replay."""
    with torch.cuda.stream(stream):
        for _ in range(replays):
            graph.replay()
        stream.synchronize()


def build_moe_sets(device, n_sets: int, seed: int = 0):
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    host = syn.moe_weights(syn.MOE_35B_A3B, seed)
    first = {k: v.to(device) for k, v in host.items()}
    sets = [mk.MoeWeights(*[first[f] for f in syn.MOE_WEIGHT_FIELDS])]
    for _ in range(n_sets - 1):
        sets.append(mk.MoeWeights(*[first[f].clone() for f in syn.MOE_WEIGHT_FIELDS]))
    return host, sets


def distinct_experts(indices: torch.Tensor) -> int:
    return int(torch.unique(indices).numel())


def bench_moe(device, batch: int, steps: int, warmup: int, sets, host_weights, peak, hold_s: float = 0.0):
    """Graph-timed MoE steps rotating over the weight sets and over different tokens."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    n_tokens = 16
    xs = [syn.hidden_states(batch, syn.MOE_35B_A3B.hidden, seed=100 + i).to(device) for i in range(n_tokens)]
    # distinct experts per token set (from an eager run), for the algorithmic byte count
    uniq = []
    for x in xs:
        _, idx, _ = mk.moe_decode(x, sets[0], top_k=8, backend="persistent")
        uniq.append(distinct_experts(idx))
    fns = [(lambda i=i: mk.moe_decode(xs[i % n_tokens], sets[i % len(sets)], top_k=8, backend="persistent")) for i in range(steps)]
    ms, graph, stream, times = time_graph(fns, warmup)
    if hold_s > 0:
        hold_load(graph, stream, max(1, int(hold_s * 1e3 / max(ms, 1e-3))))
    bytes_per_step = statistics.mean(syn.moe_algorithmic_bytes(syn.MOE_35B_A3B, batch, uniq[i % n_tokens]) for i in range(steps))
    us = ms * 1e3 / steps
    gbs = bytes_per_step / (us * 1e-6) / 1e9
    return {"us_per_step": us, "bytes_per_step": bytes_per_step, "achieved_gbs": gbs, "frac_of_measured": gbs / peak,
            "frac_of_nominal_8tbs": gbs / NOMINAL_HBM_GBS, "distinct_experts_mean": statistics.mean(uniq),
            "replays": len(times), "us_per_step_min": min(times) * 1e3 / steps, "us_per_step_max": max(times) * 1e3 / steps}


def library_dense_bar(x, dw, n, record):
    """Informational same-box bar: the dense FFN as the reference's GPU path computes it, three
    library GEMVs (`torch.nn.functional.linear`) and SiLU * mul around an fp32 RMSNorm
    (mega_kernel_qwen36/ops.py:202-218 in the reference), graph-timed like everything else.  Library
    kernels, not part of the product; reported beside the hand-written kernel's number."""
    import torch.nn.functional as F

    from mega_kernel_qwen36 import synthetic as syn

    def step():
        xf = x.float()
        xn = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * dw.norm_weight.float()).to(x.dtype)
        h = F.silu(F.linear(xn, dw.gate_weight).float()) * F.linear(xn, dw.up_weight).float()
        return (F.linear(h.to(x.dtype), dw.down_weight).float() + xf).to(x.dtype)

    step()
    ms, _, _, _ = time_graph([step] * n, 3, replays=5)
    record("dense_ffn_27b_b1_library_linear_bar", ms, n, syn.dense_algorithmic_bytes(syn.DENSE_27B, 1))


def bench_others(device, steps: int, warmup: int, peak, only=None, shape_filter=None):
    """Dense FFN, attention and linear attention at their measured shapes (rotating buffers).
    `only` ("dense", "attention", "linear" or "projection") restricts the run to one op, e.g. for a profiler."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    out = {}

    def record(name, ms, n, nbytes):
        us = ms * 1e3 / n
        gbs = nbytes / (us * 1e-6) / 1e9
        out[name] = {"us_per_step": round(us, 3), "bytes_per_step": nbytes, "achieved_gbs": round(gbs, 1),
                     "frac_of_measured": round(gbs / peak, 4), "frac_of_nominal_8tbs": round(gbs / NOMINAL_HBM_GBS, 4)}

    # dense FFN 27B: 535 MB of weights per step already exceeds the L2
    want = lambda op: only in (None, op)
    hw = syn.dense_weights(syn.DENSE_27B, 0) if want("dense") else None
    dw = mk.DenseFfnWeights(*[hw[f].to(device) for f in syn.DENSE_WEIGHT_FIELDS]) if want("dense") else None
    n = max(4, min(steps, 20))
    for batch in ((1, 8) if want("dense") else ()):
        x = syn.hidden_states(batch, syn.DENSE_27B.hidden, seed=7).to(device)
        mk.dense_ffn_decode(x, dw)
        ms, _, _, _ = time_graph([lambda: mk.dense_ffn_decode(x, dw)] * n, min(warmup, 3), replays=5)
        record(f"dense_ffn_27b_b{batch}", ms, n, syn.dense_algorithmic_bytes(syn.DENSE_27B, batch))
        if batch == 1:
            library_dense_bar(x, dw, n, record)
    del dw, hw
    torch.cuda.empty_cache()

    # attention: rotate over 4 caches (4 x 64 MiB > L2) at 32K; shorter contexts use more copies
    for seq in ((32768, 4096) if want("attention") else ()):
        copies = max(4, (3 * L2_BYTES) // (2 * seq * 2 * 256 * 2) + 1)
        t = syn.attention_tensors(1, 16, 2, 256, seq, seed=0)
        q = t["q"].to(device)
        caches = [(t["k_cache"].to(device), t["v_cache"].to(device))]
        for _ in range(copies - 1):
            caches.append((caches[0][0].clone(), caches[0][1].clone()))
        ins = [mk.FullAttentionInputs(q=q, k_cache=k, v_cache=v, scale=1.0 / 16) for k, v in caches]
        mk.full_attention_decode(ins[0])
        n = max(copies, min(steps, 200))
        fns = [(lambda i=i: mk.full_attention_decode(ins[i % copies])) for i in range(n)]
        ms, _, _, _ = time_graph(fns, warmup, replays=5)
        record(f"attention_t{seq}", ms, n, syn.attention_algorithmic_bytes(1, 16, 2, 256, seq))
        del caches, ins
        torch.cuda.empty_cache()

    # linear attention: rotate over states totalling > L2 (state is read and written: 2 x 2 MiB x B)
    for batch in ((1, 8) if want("linear") else ()):
        copies = (3 * L2_BYTES) // (batch * 32 * 128 * 128 * 4 * 2) + 2
        step = next(syn.linear_step_stream(batch, 16, 32, 128, 128, steps=1, seed=0))
        q, k, v = (step[n_].to(device) for n_ in ("q", "k", "v"))
        q32, k32 = q.repeat_interleave(2, dim=1).contiguous(), k.repeat_interleave(2, dim=1).contiguous()
        states = [syn.linear_state(batch, 32, 128, 128, seed=0).to(device)]
        for _ in range(copies - 1):
            states.append(states[0].clone())
        ins = [mk.LinearAttentionInputs(q=q32, k=k32, v=v, state=s, decay=0.9) for s in states]
        mk.linear_attention_decode(ins[0])
        n = max(copies, min(steps, 200))
        fns = [(lambda i=i: mk.linear_attention_decode(ins[i % copies])) for i in range(n)]
        ms, _, _, _ = time_graph(fns, warmup, replays=5)
        record(f"linear_attention_b{batch}", ms, n, syn.linear_algorithmic_bytes(batch, 16, 32, 128, 128))
        # resident-state variant: 64 steps per launch, the state crosses HBM twice per launch; reported per
        # step under its own name (its per-step bytes are q, k, v, out plus 1/64 of the state traffic)
        nsteps = 64
        seq = list(syn.linear_step_stream(batch, 16, 32, 128, 128, steps=nsteps, seed=1))
        qs, ks, vs = (torch.stack([s_[n_] for s_ in seq]).to(device) for n_ in ("q", "k", "v"))
        mk.linear_attention_decode_steps(qs, ks, vs, states[0], decay=0.9)
        n2 = max(4, min(copies, 16))
        fns = [(lambda i=i: mk.linear_attention_decode_steps(qs, ks, vs, states[i % copies], decay=0.9)) for i in range(n2)]
        ms, _, _, _ = time_graph(fns, min(warmup, 3), replays=5)
        per_step_bytes = (2 * batch * 32 * 128 * 128 * 4) // nsteps + batch * (2 * 16 * 128 + 2 * 32 * 128) * 2
        record(f"linear_attention_b{batch}_resident_{nsteps}steps_per_step", ms, n2 * nsteps, per_step_bytes)
        del states, ins
        torch.cuda.empty_cache()

    # decode-time projections of the 35B-A3B attention layer and the LM head: weight copies rotate so that
    # the working set exceeds the L2 (the LM head's 1 GB already does)
    if want("projection"):
        shapes = (("qkv_proj_35b", syn.QKV_35B, True, False, False), ("attn_out_proj_35b", syn.OUT_PROJ_35B, False, True, False),
                  ("lm_head_35b_argmax", syn.LM_HEAD_35B, True, False, True))
        for name, (kin, nout), norm, residual, argmax in shapes:
            if shape_filter and shape_filter not in name:
                continue
            for batch in (1, 8):
                t = syn.projection_tensors(kin, nout, batch, seed=3, norm=norm, residual=residual)
                d = {k_: v_.to(device) for k_, v_ in t.items()}
                wbytes = kin * nout * 2
                copies = max(1, (3 * L2_BYTES) // wbytes + 1) if wbytes < 3 * L2_BYTES else 2
                ws = [d["weight"]] + [d["weight"].clone() for _ in range(copies - 1)]
                call = lambda i: mk.linear_decode(d["x"], ws[i % copies], norm_weight=d.get("norm_weight"), residual=d.get("residual"),
                                                  return_argmax=argmax)
                call(0)
                n = max(copies, min(steps, 100 if wbytes < 3 * L2_BYTES else 12))
                fns = [(lambda i=i: call(i)) for i in range(n)]
                ms, _, _, _ = time_graph(fns, min(warmup, 3), replays=5)
                record(f"{name}_b{batch}", ms, n, syn.projection_algorithmic_bytes(kin, nout, batch, norm=norm, residual=residual))
                del ws, d, t
                torch.cuda.empty_cache()
    return out


def bench_e2e(device, batch: int, steps: int, warmup: int, sets):
    """Public operator with host buffers.  Per weight set one CUDA graph holds: host->device copy of
    the hidden state from pinned memory, `mk.moe_decode`, device->host copy of the output into pinned
    memory.  A timed step writes the next token into the pinned input buffer, replays the graph and
    synchronises, so the host sees the step's result."""
    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    n_tokens = 16
    hidden = syn.MOE_35B_A3B.hidden
    tokens = [syn.hidden_states(batch, hidden, seed=100 + i) for i in range(n_tokens)]
    host_x = torch.empty((batch, hidden), dtype=torch.bfloat16).pin_memory()
    host_out = torch.empty((batch, hidden), dtype=torch.bfloat16).pin_memory()
    x_dev = torch.empty((batch, hidden), dtype=torch.bfloat16, device=device)
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    graphs = []
    with torch.cuda.stream(stream):
        host_x.copy_(tokens[0])
        for w in sets:
            x_dev.copy_(host_x, non_blocking=True)
            mk.moe_decode(x_dev, w, top_k=8, backend="persistent")  # eager once: nothing allocates inside the capture
            stream.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                x_dev.copy_(host_x, non_blocking=True)
                out, _, _ = mk.moe_decode(x_dev, w, top_k=8, backend="persistent")
                host_out.copy_(out, non_blocking=True)
            graphs.append(g)

        def one(i):
            host_x.copy_(tokens[i % n_tokens])
            graphs[i % len(graphs)].replay()
            stream.synchronize()

        for i in range(warmup):
            one(i)
        stream.synchronize()
        t0 = time.perf_counter()
        for i in range(steps):
            one(i)
        dt = time.perf_counter() - t0
    h2d = batch * hidden * 2
    d2h = batch * hidden * 2
    return {"value": round(dt / steps * 1e6, 3), "unit": "us", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
            "how": "one captured graph per weight set (H2D copy of x, mk.moe_decode, D2H copy of out); per step: refill the pinned input, replay, synchronise"}


def synthetic_module():
    """The seeded input generators (`mega_kernel_qwen36/synthetic.py`) loaded as a stand-alone module,
    so that a process which only runs the CPU oracle never imports the package and with it the CUDA
    extension it is being compared with."""
    import importlib.util

    if "mega_kernel_qwen36" in sys.modules:
        from mega_kernel_qwen36 import synthetic
        return synthetic
    name = "mk36_synthetic_standalone"
    if name in sys.modules:
        return sys.modules[name]
    path = ROOT / "mega-kernel-3.6_b200" / "mega_kernel_qwen36" / "synthetic.py"
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def cpu_oracle_moe(batch: int, budget_s: float, host_weights=None):
    """The CPU oracle on the same workload, all host threads; returns (us per step, steps, cores)."""
    syn = synthetic_module()
    from oracle import decode_oracle as oracle

    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    w = host_weights if host_weights is not None else syn.moe_weights(syn.MOE_35B_A3B, 0)
    ws = [w[f] for f in syn.MOE_WEIGHT_FIELDS]
    xs = [syn.hidden_states(batch, syn.MOE_35B_A3B.hidden, seed=100 + i) for i in range(16)]
    for i in range(2):
        oracle.moe_decode(xs[i], *ws, top_k=8)
    times = []
    t_end = time.perf_counter() + budget_s
    i = 0
    while (time.perf_counter() < t_end and len(times) < 2000) or len(times) < 5:
        t0 = time.perf_counter()
        oracle.moe_decode(xs[i % 16], *ws, top_k=8)
        times.append(time.perf_counter() - t0)
        i += 1
    return statistics.median(times) * 1e6, len(times), cores


# ---------------------------------------------------------------------------------------------
def run_reference_arm(ns):
    """`--impl reference`: the reference's CPU implementation of the path (the oracle port of
    reference.py; the reference has no compiled CPU code) on the host cores, rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    us, n, cores = cpu_oracle_moe(ns.batch, budget_s=max(5.0, min(60.0, 0.05 * ns.steps)))
    line = {
        "impl": "reference",
        "metric": "us_per_decode_step", "value": round(us, 2), "unit": "us", "n_gpus": ns.gpus, "steps": ns.steps,
        "warmup": ns.warmup, "ms_per_step": round(us / 1e3, 5), "higher_is_better": False, "scaling": "strong",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": workload_config(ns.batch, ns.gpus),
        "cpu_baseline": {"value": round(us, 2), "unit": "us", "cores": cores, "kind": "port",
                         "sample": f"median of {n} steps of the same batch-{ns.batch} MoE workload (torch CPU, {cores} threads)"},
        "e2e": {"value": round(us, 2), "unit": "us", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(batch, gpus):
    """Names the workload; identical in both arms (ours / reference) for the same --batch and --gpus."""
    return {
        "workload": f"Qwen3.6-35B-A3B-shape MoE decode layer, batch {batch}: hidden 2048, 256 experts, top-8, expert "
                    "intermediate 512, shared expert 512, RMSNorm eps 1e-6, residual",
        "batch": batch,
        "parallelism": "single GPU" if gpus == 1 else f"expert parallel x{gpus} (256/{gpus} experts + 1/{gpus} of the shared expert per GPU, fp32 partial outputs summed across GPUs)",
    }


def l2_note(n_sets):
    return f"inputs larger than L2: steps rotate over {n_sets} full weight sets (the step's own bytes x sets > 126 MB) and 16 tokens"


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=20)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--sets", type=int, default=4, help="full weight sets to rotate over")
    ap.add_argument("--shape", default=None, help="with --others-only projection: only the shapes whose name contains this (e.g. lm_head)")
    ap.add_argument("--no-others", action="store_true", help="skip the context measurements of the other ops")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--others-only", choices=["dense", "attention", "linear", "projection"], default=None,
                    help="run only that op's context measurement (for profiling one kernel on a small case)")
    ap.add_argument("--collective", choices=["fused", "nccl"], default="fused",
                    help="N > 1: sum the ranks' partials inside the kernel over peer memory, or with an NCCL all-reduce")
    ns = ap.parse_args()
    ns.warmup = max(ns.warmup, 3)

    if ns.impl == "reference":
        run_reference_arm(ns)
        return

    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import synthetic as syn

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device (B200); there is no CPU path")
    if not mk.extension_available():
        raise SystemExit("the sm_100a extension is not built: run `python mega-kernel-3.6_b200/build.py`")

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    peak, peak_kind = measured_peak()

    if world > 1:
        run_expert_parallel(ns, world, rank, device, peak, peak_kind)
        return
    if ns.others_only:
        # one of the context ops alone (small enough to sit under a profiler); not a bench line
        print(json.dumps({"others_only": ns.others_only, "steps": ns.steps,
                          "others": bench_others(device, ns.steps, ns.warmup, peak, only=ns.others_only, shape_filter=ns.shape)}), flush=True)
        return

    host_weights, sets = build_moe_sets(device, ns.sets)
    sampler = ClockSampler(local_rank)
    sampler.start()
    torch.cuda.synchronize()
    res = bench_moe(device, ns.batch, ns.steps, ns.warmup, sets, host_weights, peak, hold_s=0.8)
    clocks = sampler.stop()
    clocks["sampled_over"] = "the timed graph replay and 0.8 s of further replays of the same graph"
    e2e = bench_e2e(device, ns.batch, ns.steps, ns.warmup, sets)

    others = {}
    if not ns.no_others:
        if ns.batch != 8:
            r8 = bench_moe(device, 8, max(8, ns.steps // 4), ns.warmup, sets, host_weights, peak)
            others["moe_35b_a3b_b8"] = {k: (round(v, 4) if isinstance(v, float) else v) for k, v in r8.items()}
        del sets
        torch.cuda.empty_cache()
        others.update(bench_others(device, ns.steps, ns.warmup, peak))

    cpu = None
    if not ns.no_cpu:
        us, n, cores = cpu_oracle_moe(ns.batch, budget_s=10.0, host_weights=host_weights)
        cpu = {"value": round(us, 2), "unit": "us", "cores": cores, "kind": "port",
               "sample": f"median of {n} steps of the same batch-{ns.batch} MoE workload (CPU oracle, torch, {cores} threads)"}

    us = res["us_per_step"]
    line = {
        "metric": "us_per_decode_step", "value": round(us, 3), "unit": "us", "n_gpus": 1, "steps": ns.steps, "warmup": ns.warmup,
        "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "strong", "vs_baseline": None,
        "dtype": "bf16", "data": "synthetic", "config": workload_config(ns.batch, 1), "l2": l2_note(ns.sets),
        "roofline": {"bound": "hbm", "achieved": round(res["achieved_gbs"], 1), "peak": peak, "unit": "GB/s",
                     "frac": round(res["frac_of_measured"], 4), "peak_kind": f"of {peak_kind}",
                     "frac_of_nominal_8tbs": round(res["frac_of_nominal_8tbs"], 4),
                     "algorithmic_bytes_per_launch": res["bytes_per_step"],
                     "traffic": ncu_traffic_bytes(ns.batch),
                     "value_is": f"median of {res['replays']} replays of the {ns.steps}-step graph (min {res['us_per_step_min']:.2f}, max {res['us_per_step_max']:.2f} us per step)"},
        "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": ns.steps, "clocks": clocks, "others": others,
    }
    print(json.dumps(line), flush=True)


def _parity_metrics(got: torch.Tensor, ref: torch.Tensor):
    """max-abs, relative L2 and the number of elements beyond max(2e-2, one unit in the last place of the
    output dtype) - the per-element bound the GPU tests use."""
    g, r = got.detach().cpu().double(), ref.detach().cpu().double()
    diff = (g - r).abs()
    mant = 23 if got.dtype == torch.float32 else (10 if got.dtype == torch.float16 else 7)
    ulp = torch.pow(torch.tensor(2.0, dtype=torch.float64), torch.floor(torch.log2(r.abs().clamp_min(1e-30))) - mant)
    over = int((diff > torch.maximum(torch.full_like(r, 2e-2), ulp)).sum())
    denom = float(r.norm())
    return float(diff.max()), float(diff.norm()) / (denom if denom > 0 else 1.0), over


def _same_on_all_ranks(t: torch.Tensor, world: int) -> bool:
    import torch.distributed as dist

    parts = [torch.empty_like(t) for _ in range(world)]
    dist.all_gather(parts, t.contiguous())
    return all(torch.equal(parts[0], parts[q]) for q in range(1, world))


def check_sharded_parity(ns, world, rank, device, exchange, shards, host_moe):
    """Outside the timed region: one fused step of each sharded op against the CPU oracle on the FULL
    weights (computed on rank 0), routing bit-exact, outputs bit-identical across ranks.  Collective:
    every rank calls it.  Returns the `parity` object of the bench line (rank 0) and a pass flag."""
    import torch.distributed as dist

    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import parallel, synthetic as syn
    from oracle import decode_oracle as oracle

    report = {"checked": True, "against": "CPU oracle on the full weights, rank 0", "ops": {}}
    ok = True
    # expert-parallel MoE at the timed batch and at batch 8
    for batch in sorted({ns.batch, 8}):
        x = syn.hidden_states(batch, syn.MOE_35B_A3B.hidden, seed=77 + batch)
        out, idx, rw = parallel.moe_decode_ep(x.to(device), shards[0], top_k=8, exchange=exchange)
        torch.cuda.synchronize()
        identical = _same_on_all_ranks(out, world)
        entry = {"ranks_bit_identical": identical}
        if rank == 0:
            ro, ri, rwt = oracle.moe_decode(x, *[host_moe[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=8)
            ma, rl, over = _parity_metrics(out, ro)
            entry.update({"max_abs": round(ma, 5), "rel_l2": round(rl, 6), "elements_over_bound": over,
                          "indices_exact": bool(torch.equal(idx.cpu(), ri)),
                          "route_weights_close": bool(torch.allclose(rw.cpu(), rwt, rtol=1e-4, atol=1e-5))})
            entry["pass"] = bool(over == 0 and rl <= 1e-2 and entry["indices_exact"] and entry["route_weights_close"] and identical)
            ok = ok and entry["pass"]
        report["ops"][f"moe_ep{world}_b{batch}"] = entry
    del host_moe
    # tensor-parallel dense FFN, 27B shape, batch 8
    host = syn.dense_weights(syn.DENSE_27B, 0)
    cut = parallel.shard_dense_weights(mk.DenseFfnWeights(*[host[f] for f in syn.DENSE_WEIGHT_FIELDS]), rank, world)
    local = mk.DenseFfnWeights(*[getattr(cut, f).to(device) for f in syn.DENSE_WEIGHT_FIELDS])
    x = syn.hidden_states(8, syn.DENSE_27B.hidden, seed=9)
    mk.ops._C.dense_ffn_decode_partial(x.to(device), *[getattr(local, f) for f in syn.DENSE_WEIGHT_FIELDS], 1e-6)  # local warm-up
    torch.cuda.synchronize()
    dist.barrier()
    out = parallel.dense_ffn_decode_tp(x.to(device), local, exchange=exchange)
    torch.cuda.synchronize()
    identical = _same_on_all_ranks(out, world)
    entry = {"ranks_bit_identical": identical}
    if rank == 0:
        ro = oracle.dense_ffn_decode(x, *[host[f] for f in syn.DENSE_WEIGHT_FIELDS])
        ma, rl, over = _parity_metrics(out, ro)
        entry.update({"max_abs": round(ma, 5), "rel_l2": round(rl, 6), "elements_over_bound": over})
        entry["pass"] = bool(over == 0 and rl <= 1e-2 and identical)
        ok = ok and entry["pass"]
    report["ops"][f"dense_tp{world}_b8"] = entry
    del local, cut, host
    torch.cuda.empty_cache()
    # KV-head-parallel attention (no exchange: disjoint head slices), where the head count allows this world size
    t = syn.attention_tensors(1, 16, 2, 256, 4096, seed=0)
    if 2 % world == 0:
        full = mk.FullAttentionInputs(q=t["q"], k_cache=t["k_cache"], v_cache=t["v_cache"], scale=1.0 / 16)
        mine = parallel.shard_attention_inputs(full, rank, world)
        mine = mk.FullAttentionInputs(q=mine.q.to(device), k_cache=mine.k_cache.to(device), v_cache=mine.v_cache.to(device), scale=mine.scale)
        out = parallel.full_attention_decode_kvp(mine, gather=True)
        torch.cuda.synchronize()
        entry = {"ranks_bit_identical": _same_on_all_ranks(out, world)}
        if rank == 0:
            ro = oracle.full_attention_decode(t["q"], t["k_cache"], t["v_cache"], scale=1.0 / 16)
            ma, rl, over = _parity_metrics(out, ro)
            entry.update({"max_abs": round(ma, 5), "rel_l2": round(rl, 6), "elements_over_bound": over})
            entry["pass"] = bool(over == 0 and rl <= 1e-2 and entry["ranks_bit_identical"])
            ok = ok and entry["pass"]
        report["ops"][f"attention_kvp{world}_t4096"] = entry
    flag = torch.tensor([0 if ok else 1], device=device)
    dist.all_reduce(flag)
    report["pass"] = bool(int(flag) == 0)
    return report, bool(int(flag) == 0)


def bench_attention_kvp(ns, world, rank, device, peak):
    """KV-head-parallel attention at 32K: each rank streams its own KV head(s); no exchange on the data path."""
    import torch.distributed as dist

    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import parallel, synthetic as syn

    if 2 % world != 0:
        return {}
    seq = 32768
    t = syn.attention_tensors(1, 16, 2, 256, seq, seed=0)
    full = mk.FullAttentionInputs(q=t["q"], k_cache=t["k_cache"], v_cache=t["v_cache"], scale=1.0 / 16)
    cut = parallel.shard_attention_inputs(full, rank, world)
    q = cut.q.to(device)
    caches = [(cut.k_cache.to(device), cut.v_cache.to(device))]
    per_rank = 2 * seq * (2 // world) * 256 * 2
    while per_rank * len(caches) < 3 * L2_BYTES:
        caches.append((caches[0][0].clone(), caches[0][1].clone()))
    ins = [mk.FullAttentionInputs(q=q, k_cache=k, v_cache=v, scale=cut.scale) for k, v in caches]
    mk.full_attention_decode(ins[0])
    n = max(len(ins), min(ns.steps, 100))
    torch.cuda.synchronize()
    dist.barrier()
    ms, _, _, _ = time_graph([(lambda i=i: mk.full_attention_decode(ins[i % len(ins)])) for i in range(n)], ns.warmup, replays=5)
    tms = torch.tensor([ms], device=device)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    us = float(tms) * 1e3 / n
    nbytes = syn.attention_algorithmic_bytes(1, 16, 2, 256, seq)
    gbs = nbytes / (us * 1e-6) / 1e9
    del caches, ins
    torch.cuda.empty_cache()
    return {f"attention_kvp{world}_t{seq}": {"us_per_step": round(us, 3), "bytes_per_step": nbytes, "achieved_gbs": round(gbs, 1),
                                             "frac_of_measured": round(gbs / (peak * world), 4)}}


def bench_moe_ep_batch(ns, world, rank, device, shards, exchange, peak, batch: int):
    """The expert-parallel MoE step at another batch size, graph-timed like the headline (max over ranks)."""
    import torch.distributed as dist

    from mega_kernel_qwen36 import parallel, synthetic as syn

    n_tokens = 8
    xs = [syn.hidden_states(batch, syn.MOE_35B_A3B.hidden, seed=300 + i).to(device) for i in range(n_tokens)]
    uniq = []
    for i in range(n_tokens):
        _, idx, _ = parallel.moe_decode_ep(xs[i], shards[i % len(shards)], top_k=8, exchange=exchange)
        uniq.append(distinct_experts(idx))
    n = max(8, min(ns.steps, 64))
    torch.cuda.synchronize()
    dist.barrier()
    fns = [(lambda i=i: parallel.moe_decode_ep(xs[i % n_tokens], shards[i % len(shards)], top_k=8, exchange=exchange)) for i in range(n)]
    ms, _, _, _ = time_graph(fns, 3, replays=5)
    tms = torch.tensor([ms], device=device)
    dist.all_reduce(tms, op=dist.ReduceOp.MAX)
    us = float(tms) * 1e3 / n
    nbytes = statistics.mean(syn.moe_algorithmic_bytes(syn.MOE_35B_A3B, batch, uniq[i % n_tokens]) for i in range(n))
    gbs = nbytes / (us * 1e-6) / 1e9
    dist.barrier()
    return {f"moe_35b_a3b_ep{world}_b{batch}": {"us_per_step": round(us, 3), "bytes_per_step": nbytes, "achieved_gbs": round(gbs, 1),
                                                "frac_of_measured": round(gbs / (peak * world), 4)}}


def bench_dense_tp(ns, world, rank, device, exchange, peak):
    """Tensor-parallel dense FFN (27B shape) on the same ranks: one kernel per step per GPU with the
    cross-GPU sum inside, graph-timed like the headline.  Collective: every rank calls it."""
    import torch.distributed as dist

    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import parallel, synthetic as syn

    out = {}
    host = syn.dense_weights(syn.DENSE_27B, 0)
    cut = parallel.shard_dense_weights(mk.DenseFfnWeights(*[host[f] for f in syn.DENSE_WEIGHT_FIELDS]), rank, world)
    local = mk.DenseFfnWeights(*[getattr(cut, f).to(device) for f in syn.DENSE_WEIGHT_FIELDS])
    copies = [local]
    per_rank = syn.dense_algorithmic_bytes(syn.DENSE_27B, 1) // world
    while per_rank * len(copies) < 3 * L2_BYTES:  # rotate so that the working set exceeds the L2
        copies.append(mk.DenseFfnWeights(*[getattr(local, f).clone() for f in syn.DENSE_WEIGHT_FIELDS]))
    del host, cut
    n = max(len(copies), min(ns.steps, 40))
    for batch in (1, 8):
        x = syn.hidden_states(batch, syn.DENSE_27B.hidden, seed=7).to(device)
        mk.ops._C.dense_ffn_decode_partial(x, *[getattr(local, f) for f in syn.DENSE_WEIGHT_FIELDS], 1e-6)  # local warm-up
        torch.cuda.synchronize()
        dist.barrier()
        fns = [(lambda i=i: parallel.dense_ffn_decode_tp(x, copies[i % len(copies)], exchange=exchange)) for i in range(n)]
        ms, _, _, _ = time_graph(fns, 3, replays=5)
        t = torch.tensor([ms], device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        us = float(t) * 1e3 / n
        nbytes = syn.dense_algorithmic_bytes(syn.DENSE_27B, batch)
        gbs = nbytes / (us * 1e-6) / 1e9
        out[f"dense_ffn_27b_tp{world}_b{batch}"] = {"us_per_step": round(us, 3), "bytes_per_step": nbytes, "achieved_gbs": round(gbs, 1),
                                                   "frac_of_measured": round(gbs / (peak * world), 4)}
        dist.barrier()
    return out


def run_expert_parallel(ns, world, rank, device, peak, peak_kind):
    """N ranks, one per GPU: expert-parallel MoE step, the ranks' partial outputs summed inside the
    kernel over peer memory (or, with --collective nccl, by an all-reduce after it)."""
    import torch.distributed as dist

    import mega_kernel_qwen36 as mk
    from mega_kernel_qwen36 import parallel, synthetic as syn

    dist.init_process_group("nccl", device_id=device)
    host = syn.moe_weights(syn.MOE_35B_A3B, 0)
    full = mk.MoeWeights(*[host[f] for f in syn.MOE_WEIGHT_FIELDS])
    shards = []
    base = parallel.shard_moe_weights(full, rank, world)
    first = mk.MoeWeights(*[getattr(base.weights, f).to(device) for f in syn.MOE_WEIGHT_FIELDS])
    shards.append(parallel.MoeShard(first, base.expert_base, rank, world))
    for _ in range(ns.sets - 1):
        shards.append(parallel.MoeShard(mk.MoeWeights(*[getattr(first, f).clone() for f in syn.MOE_WEIGHT_FIELDS]),
                                        base.expert_base, rank, world))
    host_moe = host if rank == 0 else None  # rank 0 keeps the full weights for the parity check
    del host, full
    n_tokens = 16
    xs = [syn.hidden_states(ns.batch, syn.MOE_35B_A3B.hidden, seed=100 + i).to(device) for i in range(n_tokens)]

    # a local (non-collective) launch first: module loading on one rank must not eat into the
    # bounded waits of the others
    w0 = shards[0].weights
    mk.ops._C.moe_decode_partial(xs[0], *[getattr(w0, f) for f in syn.MOE_WEIGHT_FIELDS], 1e-6, 8, shards[0].expert_base)
    torch.cuda.synchronize()
    exchange = None if ns.collective == "nccl" else parallel.PeerExchange(device)
    dist.barrier()

    def step(i):
        return parallel.moe_decode_ep(xs[i % n_tokens], shards[i % len(shards)], top_k=8, exchange=exchange)

    # distinct experts per token set (identical on all ranks), for the algorithmic byte count
    uniq = []
    for i in range(n_tokens):
        _, idx, _ = step(i)
        uniq.append(distinct_experts(idx))

    sampler = ClockSampler(device.index)
    if rank == 0:
        sampler.start()
    if exchange is not None:
        # one launch per step and nothing else: K steps in one CUDA graph, as on a single GPU; the ranks
        # meet inside every step, so the replays stay in lock-step
        fns = [(lambda i=i: step(i)) for i in range(ns.steps)]
        dist.barrier()
        ms_local, graph, stream, _ = time_graph(fns, ns.warmup, replays=1)
        torch.cuda.synchronize()
        dist.barrier()
        with torch.cuda.stream(stream):
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            start.record(stream)
            graph.replay()
            end.record(stream)
            end.synchronize()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        # the same number of further replays on every rank, for the clock sampler
        worst = ms.clone()
        dist.all_reduce(worst, op=dist.ReduceOp.MAX)
        hold_load(graph, stream, max(1, int(800.0 / max(float(worst), 1e-3))))
        timing = "CUDA graph of all steps (one kernel per step per GPU, cross-GPU sum inside the kernel), CUDA events, max over ranks"
    else:
        for i in range(ns.warmup):
            step(i)
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(ns.steps):
            step(i)
        end.record()
        torch.cuda.synchronize()
        ms = torch.tensor([start.elapsed_time(end)], device=device)
        timing = "eager launches (kernel + NCCL all-reduce + residual per step), CUDA events, max over ranks"
    dist.barrier()
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    e2e = None
    host_x = [x.cpu().pin_memory() for x in xs]
    host_out = torch.empty_like(host_x[0]).pin_memory()
    x_dev = torch.empty_like(xs[0])
    torch.cuda.synchronize()
    dist.barrier()
    t0 = time.perf_counter()
    for i in range(ns.steps):
        x_dev.copy_(host_x[i % n_tokens], non_blocking=True)
        out, _, _ = parallel.moe_decode_ep(x_dev, shards[i % len(shards)], top_k=8, exchange=exchange)
        host_out.copy_(out, non_blocking=True)
        torch.cuda.current_stream().synchronize()
    torch.cuda.synchronize()
    dt = torch.tensor([time.perf_counter() - t0], device=device)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    nbytes = ns.batch * syn.MOE_35B_A3B.hidden * 2
    e2e = {"value": round(float(dt) / ns.steps * 1e6, 3), "unit": "us", "h2d_bytes_per_step": nbytes, "d2h_bytes_per_step": nbytes}
    others = {}
    parity = {"checked": False, "why": "the NCCL variant is the plain collective path; the parity check covers the fused exchange"}
    parity_ok = True
    if exchange is not None:
        parity, parity_ok = check_sharded_parity(ns, world, rank, device, exchange, shards, host_moe)
    if not ns.no_others and exchange is not None:
        if ns.batch != 8:
            others.update(bench_moe_ep_batch(ns, world, rank, device, shards, exchange, peak, 8))
        del shards
        torch.cuda.empty_cache()
        others.update(bench_dense_tp(ns, world, rank, device, exchange, peak))
        others.update(bench_attention_kvp(ns, world, rank, device, peak))
    if rank == 0:
        us = float(ms) * 1e3 / ns.steps
        nbytes_alg = statistics.mean(syn.moe_algorithmic_bytes(syn.MOE_35B_A3B, ns.batch, uniq[i % n_tokens]) for i in range(ns.steps))
        gbs = nbytes_alg / (us * 1e-6) / 1e9
        line = {
            "metric": "us_per_decode_step", "value": round(us, 3), "unit": "us", "n_gpus": world, "steps": ns.steps,
            "warmup": ns.warmup, "ms_per_step": round(us / 1e3, 6), "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(ns.batch, world), "l2": l2_note(ns.sets),
            "roofline": {"bound": "hbm", "achieved": round(gbs, 1), "peak": peak * world, "unit": "GB/s",
                         "frac": round(gbs / (peak * world), 4), "peak_kind": f"of {peak_kind} x {world} GPUs",
                         "algorithmic_bytes_per_launch": nbytes_alg, "traffic": None},
            "cpu_baseline": None, "e2e": e2e, "gpu_launches": ns.steps, "clocks": clocks,
            "timing": timing, "parity": parity, "others": others,
        }
        print(json.dumps(line), flush=True)
    torch.cuda.synchronize()
    dist.barrier()
    if exchange is not None:
        exchange.close()
    dist.destroy_process_group()
    if not parity_ok:
        raise SystemExit("bench.py: a sharded op failed its parity check (see `parity` in the line above)")


if __name__ == "__main__":
    main()
