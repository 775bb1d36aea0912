"""Shared pytest setup: import paths, the gpu marker, and GPU-availability
gating (tests marked gpu are skipped where no CUDA device is visible)."""

import pathlib
import sys

import pytest

ROOT = pathlib.Path(__file__).resolve().parent.parent
for path in (ROOT, ROOT / "flywheel-tpu_b200", ROOT / "tests", ROOT / "tests" / "golden"):
    if str(path) not in sys.path:
        sys.path.insert(0, str(path))


def pytest_configure(config):
    config.addinivalue_line(
        "markers", "gpu: needs a CUDA device (run on a B200 box)")


def cuda_available():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:  # pylint: disable=broad-except
        return False


def pytest_collection_modifyitems(config, items):
    if cuda_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device visible")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)
