"""Expert-parallel MoE, tensor-parallel dense FFN and KV-head-parallel attention on 2, 4 and 8 GPUs,
with the cross-GPU sum fused into the kernels' epilogue (peer stores over NVLink, bounded waits).

Every world size that the machine has GPUs for is run; the others are skipped.  The ranks are separate
processes (torchrun), one per GPU: kernels that wait on one another must never share a GPU.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


@pytest.mark.parametrize("world", [2, 4, 8])
def test_fused_exchange(world, cuda_device):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29561 + world), str(ROOT / "tests" / "multi_gpu_worker.py")]
    proc = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=1200)
    tail = (proc.stdout + proc.stderr)[-4000:]
    assert proc.returncode == 0 and "MULTI_GPU_OK" in proc.stdout, tail
