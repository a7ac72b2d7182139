import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def model_dirs(tmp_path_factory):
    """Model folders of the tiny configurations, made with the random-weights mode in a
    temporary folder."""
    from tiny_configs import make_all
    return make_all(tmp_path_factory.mktemp("models"))


@pytest.fixture()
def cpu_backend():
    """Install the torch-CPU test double of the kernel library for a test of host logic."""
    from cpu_backend import CpuBackend
    from nimbus_infer_rs_b200.csrc import ops
    b = CpuBackend()
    ops.set_backend(b)
    yield b
    ops.set_backend(None)
