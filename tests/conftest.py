import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA GPU (B200)")
    config.addinivalue_line("markers", "multigpu: test needs more than one GPU")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session", autouse=True)
def _native_built():
    """Build the native extension once (cross-compiles without a GPU)."""
    from planmoe_b200.ops import native
    if not native.available():
        from planmoe_b200.utils import build
        build.build()
        native._ERR = None
        native._try_load()
    return native.available()
