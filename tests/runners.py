"""Runs one golden case through the CPU oracle or through the CUDA package; loads fixtures."""

from __future__ import annotations

import functools
from pathlib import Path
from typing import Dict

import numpy as np
import torch

from golden_cases import CASES_BY_NAME, STATE_STRIDE, Case, checksum
from mega_kernel_qwen36 import synthetic as syn
from oracle import decode_oracle as oracle

GOLDEN_DIR = Path(__file__).resolve().parent / "golden"


def load_golden(name: str) -> Dict[str, np.ndarray]:
    with np.load(GOLDEN_DIR / f"{name}.npz") as z:
        return {k: z[k] for k in z.files}


@functools.lru_cache(maxsize=2)
def _cached_inputs(name: str):
    return CASES_BY_NAME[name].build()


def build_inputs(case: Case):
    """Inputs of a case; the two most recent are cached (the big MoE draws take ~10 s)."""
    return _cached_inputs(case.name)


def fingerprint(case: Case, spec) -> np.ndarray:
    if case.op == "moe":
        t = spec["tensors"]
        fp = [checksum(t["x"]), checksum(t["router_weight"]), checksum(t["expert_down"]), checksum(t["shared_up"])]
    elif case.op == "dense":
        t = spec["tensors"]
        fp = [checksum(t["x"]), checksum(t["gate_weight"]), checksum(t["down_weight"])]
    elif case.op == "attention":
        t = spec["tensors"]
        fp = [checksum(t["q"]), checksum(t["k_cache"]), checksum(t["v_cache"])]
    else:
        fp = ([checksum(spec["state"])] + [checksum(s["v"]) for s in spec["steps"]])[:8]
    return np.asarray(fp, dtype=np.float64)


def assert_same_inputs(case: Case, spec, golden) -> None:
    np.testing.assert_allclose(fingerprint(case, spec), golden["fingerprint"], rtol=1e-12, atol=0,
                               err_msg=f"{case.name}: seeded inputs differ from the ones the fixture was made with")


# ---------------------------------------------------------------------------------------------
def run_oracle(case: Case, spec) -> Dict[str, torch.Tensor]:
    if case.op == "moe":
        t = spec["tensors"]
        y, idx, w = oracle.moe_decode(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=spec["top_k"])
        return {"out": y, "indices": idx, "weights": w}
    if case.op == "dense":
        t = spec["tensors"]
        return {"out": oracle.dense_ffn_decode(t["x"], *[t[f] for f in syn.DENSE_WEIGHT_FIELDS])}
    if case.op == "attention":
        t = spec["tensors"]
        return {"out": oracle.full_attention_decode(t["q"], t["k_cache"], t["v_cache"], scale=spec["scale"])}
    if case.op == "linear":
        state = spec["state"]
        outs, norms = [], []
        for step in spec["steps"]:
            q = step["q"].repeat_interleave(spec["expand"], dim=1)
            k = step["k"].repeat_interleave(spec["expand"], dim=1)
            y, state = oracle.linear_attention_decode(q, k, step["v"], state, decay=spec["decay"])
            outs.append(y)
            norms.append(float(state.double().norm()))
        return {"outs": outs, "state_norms": norms, "state": state}
    raise ValueError(case.op)


def run_cuda(case: Case, spec, device) -> Dict[str, torch.Tensor]:
    import mega_kernel_qwen36 as mk

    if case.op == "moe":
        t = {k: v.to(device) for k, v in spec["tensors"].items()}
        w = mk.MoeWeights(*[t[f] for f in syn.MOE_WEIGHT_FIELDS])
        y, idx, rw = mk.moe_decode(t["x"], w, top_k=spec["top_k"], backend="persistent")
        return {"out": y.cpu(), "indices": idx.cpu(), "weights": rw.cpu()}
    if case.op == "dense":
        t = {k: v.to(device) for k, v in spec["tensors"].items()}
        w = mk.DenseFfnWeights(*[t[f] for f in syn.DENSE_WEIGHT_FIELDS])
        return {"out": mk.dense_ffn_decode(t["x"], w).cpu()}
    if case.op == "attention":
        t = {k: v.to(device) for k, v in spec["tensors"].items()}
        y = mk.full_attention_decode(mk.FullAttentionInputs(q=t["q"], k_cache=t["k_cache"], v_cache=t["v_cache"],
                                                            scale=spec["scale"]))
        return {"out": y.cpu()}
    if case.op == "linear":
        state = spec["state"].to(device)
        outs, norms = [], []
        for step in spec["steps"]:
            q = step["q"].repeat_interleave(spec["expand"], dim=1).to(device)
            k = step["k"].repeat_interleave(spec["expand"], dim=1).to(device)
            y, state = mk.linear_attention_decode(mk.LinearAttentionInputs(q=q, k=k, v=step["v"].to(device),
                                                                           state=state, decay=spec["decay"]))
            outs.append(y.cpu())
            norms.append(float(state.double().norm()))
        return {"outs": outs, "state_norms": norms, "state": state.cpu()}
    raise ValueError(case.op)


def golden_state_sample(state: torch.Tensor) -> np.ndarray:
    return state[..., ::STATE_STRIDE, ::STATE_STRIDE].contiguous().cpu().numpy()
