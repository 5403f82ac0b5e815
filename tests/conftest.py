"""pytest configuration: registers the ``gpu`` marker and skips GPU tests without a device."""

import pytest
import torch


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device (B200, sm_100a)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(autouse=True)
def _check_kernel_errors(request):
    """After every GPU test make sure no kernel recorded a bounded-wait failure."""
    yield
    if "gpu" in request.keywords and torch.cuda.is_available():
        from lorafusion_b200.ops import _native as nv

        nv.check_device_errors()
