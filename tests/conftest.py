import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")
    config.addinivalue_line("markers", "expects_device_status: the test provokes and reads the device status word itself")


@pytest.fixture(scope="session")
def hl_ctx():
    """One hl_ctx for the whole GPU session, on torch's current stream."""
    import torch

    import hippo_leap_b200 as hl

    if not torch.cuda.is_available():
        pytest.fail("GPU test selected but no CUDA device is visible")
    torch.cuda.set_device(0)
    ctx = hl.Context(0, torch.cuda.current_stream())
    yield ctx
    ctx.close()


@pytest.fixture(autouse=True)
def _device_status_clean(request):
    """After every GPU test the device status word must be clean (no timeout / bounds hit)."""
    yield
    if "hl_ctx" in request.fixturenames and "expects_device_status" not in request.keywords:
        ctx = request.getfixturevalue("hl_ctx")
        code, detail = ctx.device_status()
        assert code == 0, f"device status {code} (detail {detail}) left by {request.node.name}"
