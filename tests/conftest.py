import os
import sys

import pytest
import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


try:
    # Property tests draw the same examples on every run (a plain `pytest` is reproducible); set
    # PXL_HYPOTHESIS_RANDOM=1 (optionally with --hypothesis-seed) to hunt with fresh ones.
    from hypothesis import settings as _hyp_settings

    _hyp_settings.register_profile("repo", derandomize=not os.environ.get("PXL_HYPOTHESIS_RANDOM"), deadline=None,
                                   database=None)
    _hyp_settings.load_profile("repo")
except ImportError:
    pass


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
