import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def _ensure_native_libraries():
    """The package refuses to import without its libraries (there is no fallback), so a fresh
    checkout builds them before the first test module is collected. Up-to-date libraries are left
    alone."""
    os.environ["B200TBE_BUILDING"] = "1"
    try:
        from torchlib_xpu_b200 import _build

        _build.build_all()
    finally:
        del os.environ["B200TBE_BUILDING"]


_ensure_native_libraries()


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


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
