import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


# Multi-GPU tests that have not yet completed a run on real hardware (GPU slots were unavailable when they
# were written) only run on request, so that a first-run surprise cannot stop the rest of the suite.
unvalidated = pytest.mark.skipif(not os.environ.get("XPOOL_RUN_UNVALIDATED"),
                                 reason="not yet validated on a multi-GPU box; set XPOOL_RUN_UNVALIDATED=1 to run")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a real B200 (run with -m gpu)")


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
