import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200) and the built CUDA library")


def pytest_collection_modifyitems(config, items):
    try:
        import torch
        has_gpu = torch.cuda.is_available()
    except Exception:  # pragma: no cover
        has_gpu = False
    if has_gpu:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """Write the achieved parity errors of this session where FB_PARITY_REPORT points (optional)."""
    path = os.environ.get("FB_PARITY_REPORT")
    if not path:
        return
    import json
    from tests import helpers
    with open(path, "w") as f:
        json.dump(helpers.ACHIEVED, f, indent=1, sort_keys=True)
