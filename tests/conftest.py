"""pytest configuration: the ``gpu`` marker and import paths.

Tests marked ``gpu`` need a B200 and the built extension; everything else runs on CPU.
"""

import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
PACKAGE_DIR = ROOT / "mega-kernel-3.6_b200"
for p in (str(ROOT), str(PACKAGE_DIR)):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built sm_100a extension")


def pytest_sessionfinish(session, exitstatus):
    """Writes the parity figures of the session (plain max-abs, relative L2 and the number of elements
    beyond a flat 2e-2 per comparison) to the file named by MK36_PARITY_REPORT, when that is set."""
    import json
    import os

    target = os.environ.get("MK36_PARITY_REPORT")
    if not target:
        return
    try:
        import parity

        if parity.REPORT:
            Path(target).write_text(json.dumps(parity.REPORT, indent=1, sort_keys=True))
    except Exception:  # a report is a convenience, never a reason to fail the session
        pass


@pytest.fixture(scope="session")
def cuda_device():
    import torch

    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran without a CUDA device")
    import mega_kernel_qwen36 as mk

    if not mk.extension_available():
        pytest.fail("the sm_100a extension is not built; GPU tests never fall back to PyTorch")
    return torch.device("cuda:0")
