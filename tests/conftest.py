import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
os.environ.setdefault("WANDB_MODE", "disabled")

# the upstream tree, when it is mounted next to this repository (or named by PD_REFERENCE_ROOT)
_REF_ROOT = Path(os.environ.get("PD_REFERENCE_ROOT", ROOT.parent / "reference"))
REFERENCE_CONFIGS = _REF_ROOT / "param_decomp" / "param_decomp" / "experiments"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")
    config.addinivalue_line("markers", "slow: longer-running CPU test")


@pytest.fixture(scope="session")
def reference_configs():
    if not REFERENCE_CONFIGS.exists():
        pytest.skip("reference tree not mounted")
    return REFERENCE_CONFIGS


@pytest.fixture()
def cuda():
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    return torch.device("cuda", 0)
