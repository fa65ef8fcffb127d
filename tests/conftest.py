import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    # tests marked gpu are skipped, not failed, on a machine without a device
    try:
        import torch
        have = torch.cuda.is_available()
    except Exception:
        have = False
    if have:
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def pytest_sessionfinish(session, exitstatus):
    """With GARUDA_B200_RECORD_ERRORS=<file>: the largest difference every configuration showed
    against the plain implementation, as the tolerances in tests/helpers.py are derived from it."""
    path = os.environ.get("GARUDA_B200_RECORD_ERRORS")
    if not path:
        return
    import json
    from tests import helpers
    with open(path, "w") as f:
        json.dump(dict(sorted(helpers.OBSERVED.items())), f, indent=1)
