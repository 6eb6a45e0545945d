import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def pkg():
    import __graft_entry__ as ge
    return ge.load_package()


@pytest.fixture(scope="session")
def ctx(pkg):
    """One context on cuda:0 using torch's current stream.  Fails (does not skip)
    when the library or the GPU is missing: GPU tests must not pass on a fallback."""
    import torch
    assert torch.cuda.is_available(), "GPU tests need a CUDA device"
    c = pkg.Context(0)
    c.use_torch_stream()
    yield c
    c.close()


@pytest.fixture(scope="session")
def golden_ops():
    import numpy as np
    return np.load(ROOT / "tests" / "golden" / "ops_ref.npz")
