"""Shared pytest configuration: the ``gpu`` marker, import paths, fixtures."""

import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


def pytest_collection_modifyitems(config, items):
    import torch

    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device in this process")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def golden():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "sdpa_golden.pt")
    return torch.load(path, weights_only=False)["cases"]


@pytest.fixture(scope="session")
def golden_bwd():
    import torch

    path = os.path.join(ROOT, "tests", "golden", "sdpa_bwd_golden.pt")
    return torch.load(path, weights_only=False)["cases"]


@pytest.fixture(autouse=True)
def _checked_build_verdict(request):
    """Under ``B200_SDPA_CHECKED=1`` (the bounds-checking build of the library) every GPU test also
    fails when a kernel recorded an index, scratch-slot or tensor-memory column violation."""
    yield
    if os.environ.get("B200_SDPA_CHECKED", "0") not in ("", "0") and "gpu" in request.keywords:
        import torch

        if torch.cuda.is_available():
            import torch_neuronx_b200 as T

            T.check_device_status()
