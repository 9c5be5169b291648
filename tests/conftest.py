import os
import sys
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

os.environ.setdefault("MASTER_ADDR", "127.0.0.1")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200)")
    config.addinivalue_line("markers", "multigpu(n): needs at least n CUDA devices")
    config.addinivalue_line("markers", "slow: long-running")


def pytest_collection_modifyitems(config, items):
    have = torch.cuda.is_available()
    ndev = torch.cuda.device_count() if have else 0
    for item in items:
        if "gpu" in item.keywords and not have:
            item.add_marker(pytest.mark.skip(reason="no CUDA device"))
        m = item.get_closest_marker("multigpu")
        if m is not None and ndev < int(m.args[0]):
            item.add_marker(pytest.mark.skip(reason=f"needs {m.args[0]} GPUs, have {ndev}"))


@pytest.fixture(autouse=True)
def _seed():
    torch.manual_seed(0)
    yield


@pytest.fixture(autouse=True)
def _kernel_status_clean(request):
    """After every GPU test the library status block must report no timed-out wait."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from hybrid_model_factory_b200.ops import _lib
        if _lib.kernels_available():
            _lib.assert_status_ok()
