"""Shared pytest setup: markers, import path, and the GPU gate."""

import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
if str(ROOT / "tests") not in sys.path:
    sys.path.insert(0, str(ROOT / "tests"))


def pytest_configure(config):
    config.addinivalue_line(
        "markers", "gpu: needs a CUDA device (run with -m gpu on a B200)"
    )


def pytest_collection_modifyitems(config, items):
    """GPU tests never run silently on a machine without a device."""
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


@pytest.fixture(scope="session")
def native_library():
    """The built C-ABI library; building is part of the test session."""
    from swage_b200 import _build, _native

    _build.build_library()
    return _native.library()
