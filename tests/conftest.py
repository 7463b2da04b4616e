import os
import sys

import pytest

# a stuck worker must not stall a test run for the production shutdown budget (600 s per worker)
os.environ.setdefault("FLEXKV_WORKER_SHUTDOWN_TIMEOUT_S", "15")
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")
    config.addinivalue_line("markers", "multigpu: needs at least two CUDA devices")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        ngpu = torch.cuda.device_count() if torch.cuda.is_available() else 0
    except Exception:  # noqa: BLE001
        ngpu = 0
    for item in items:
        if "multigpu" in item.keywords and ngpu < 2:
            item.add_marker(pytest.mark.skip(reason="needs >= 2 GPUs"))
        elif "gpu" in item.keywords and ngpu < 1:
            item.add_marker(pytest.mark.skip(reason="needs a GPU"))


@pytest.fixture(scope="session")
def native():
    from flexkv_b200 import _native
    return _native.C
