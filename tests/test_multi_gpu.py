"""Expert-parallel MoE and tensor-parallel dense FFN on two GPUs, with the cross-GPU sum fused
into the kernels' epilogue (peer stores over NVLink, bounded waits).

Needs two GPUs in one box; skipped on a single-GPU machine.  The ranks are separate processes
(torchrun), one per GPU: kernels that wait on one another must never share a GPU.
"""

import os
import subprocess
import sys
from pathlib import Path

import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = Path(__file__).resolve().parent.parent


def test_fused_exchange_two_gpus(cuda_device):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    env = dict(os.environ)
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29561", str(ROOT / "tests" / "multi_gpu_worker.py")]
    proc = subprocess.run(cmd, cwd=str(ROOT), env=env, capture_output=True, text=True, timeout=900)
    tail = (proc.stdout + proc.stderr)[-4000:]
    assert proc.returncode == 0 and "MULTI_GPU_OK" in proc.stdout, tail
