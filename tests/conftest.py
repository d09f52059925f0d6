import importlib
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    return importlib.import_module("deep-learning-framework_b200")


@pytest.fixture(scope="session")
def vm(pkg):
    return pkg.vmath


@pytest.fixture(scope="session")
def port():
    import oracle
    return oracle.Oracle("port")


@pytest.fixture(scope="session")
def torch_cuda():
    import torch
    if not torch.cuda.is_available():
        pytest.fail("a test marked gpu ran on a machine without CUDA")
    torch.cuda.set_device(0)
    return torch
