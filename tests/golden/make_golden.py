"""Generates tests/golden/*.npz by running the reference's own ``mega_kernel_qwen36/reference.py``.

    python tests/golden/make_golden.py [--reference /path/to/Mega-Kernel-3.6] [--only NAME ...]

The reference checkout is imported, not copied: ``moe_decode_reference`` (reference.py:16-62),
``dense_ffn_decode_reference`` (:65-88), ``full_attention_decode_reference`` (:117-145) and
``linear_attention_decode_reference`` (:148-166) are called on the seeded inputs of
tests/golden_cases.py, on CPU, with the same tensors (and dtypes) the CUDA kernels get.
Outputs are stored as float32 (exact for bf16 / fp16 values) together with fingerprints of the
inputs, so that a test on a machine without the reference can tell a wrong kernel from a
different random stream.
"""

from __future__ import annotations

import argparse
import importlib.util
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "mega-kernel-3.6_b200"))
sys.path.insert(0, str(ROOT / "tests"))

from golden_cases import CASES, STATE_STRIDE, checksum  # noqa: E402
from mega_kernel_qwen36 import synthetic as syn  # noqa: E402


def load_reference(root: Path):
    path = root / "mega_kernel_qwen36" / "reference.py"
    spec = importlib.util.spec_from_file_location("mk36_upstream_reference", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def run_case(ref, case) -> dict:
    spec = case.build()
    out = {}
    if case.op == "moe":
        t = spec["tensors"]
        y, idx, w = ref.moe_decode_reference(t["x"], *[t[f] for f in syn.MOE_WEIGHT_FIELDS], top_k=spec["top_k"])
        out = {"out": y.float().numpy(), "indices": idx.numpy(), "weights": w.numpy()}
        fp = [checksum(t["x"]), checksum(t["router_weight"]), checksum(t["expert_down"]), checksum(t["shared_up"])]
    elif case.op == "dense":
        t = spec["tensors"]
        y = ref.dense_ffn_decode_reference(t["x"], *[t[f] for f in syn.DENSE_WEIGHT_FIELDS])
        out = {"out": y.float().numpy()}
        fp = [checksum(t["x"]), checksum(t["gate_weight"]), checksum(t["down_weight"])]
    elif case.op == "attention":
        t = spec["tensors"]
        y = ref.full_attention_decode_reference(t["q"], t["k_cache"], t["v_cache"], scale=spec["scale"])
        out = {"out": y.float().numpy()}
        fp = [checksum(t["q"]), checksum(t["k_cache"]), checksum(t["v_cache"])]
    elif case.op == "linear":
        state = spec["state"]
        fp = [checksum(state)]
        outs, norms = [], []
        n_steps = len(spec["steps"])
        keep = sorted({0, 1, n_steps // 2, n_steps - 1} & set(range(n_steps)))
        for si, step in enumerate(spec["steps"]):
            q = step["q"].repeat_interleave(spec["expand"], dim=1)
            k = step["k"].repeat_interleave(spec["expand"], dim=1)
            y, state = ref.linear_attention_decode_reference(q, k, step["v"], state, decay=spec["decay"])
            if si in keep:
                outs.append(y.float().numpy())
            norms.append(float(state.double().norm()))
            fp.append(checksum(step["v"]))
        out = {
            "outs": np.stack(outs),          # outputs of the steps listed in out_steps
            "out_steps": np.asarray(keep, dtype=np.int64),
            "state_norms": np.asarray(norms, dtype=np.float64),
            "state_sample": state[..., ::STATE_STRIDE, ::STATE_STRIDE].contiguous().numpy(),
            "state_sum": np.asarray(float(state.double().sum())),
        }
        fp = fp[:8]
    else:
        raise ValueError(case.op)
    out["fingerprint"] = np.asarray(fp, dtype=np.float64)
    return out


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="root of a checkout of the reference project")
    ap.add_argument("--only", nargs="*", default=None)
    ns = ap.parse_args()
    ref = load_reference(Path(ns.reference))
    torch.manual_seed(0)
    for case in CASES:
        if ns.only and case.name not in ns.only:
            continue
        data = run_case(ref, case)
        np.savez_compressed(HERE / f"{case.name}.npz", **data)
        size = (HERE / f"{case.name}.npz").stat().st_size
        print(f"{case.name}: {size} bytes", flush=True)


if __name__ == "__main__":
    main()
