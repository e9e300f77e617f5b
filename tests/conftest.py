"""Shared pytest configuration: the ``gpu`` marker and helpers used by both suites."""
import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
GOLDEN = ROOT / "tests" / "golden"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device of compute capability 10.x (B200)")


@pytest.fixture(scope="session")
def host_golden():
    return json.loads((GOLDEN / "reference_host_logic.json").read_text())


@pytest.fixture(scope="session")
def step_golden():
    import torch
    return torch.load(GOLDEN / "reference_muon_step.pt")


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    major, _ = torch.cuda.get_device_capability(0)
    if major != 10:
        pytest.fail("GPU tests need an sm_100a device")
    from i8muon_b200.build import build
    build()
    return torch.device("cuda", 0)
