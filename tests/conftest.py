import os
import sys

import numpy as np
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


@pytest.fixture(scope="session")
def wmma_known_answers():
    """The two fp16 x fp16 -> fp32 16x16x16 products whose answers the reference's tests/integration_wmma.nim derives in
    closed form: A[r][k] = 100 r + k, B[k][c] = k + 1  =>  C[r][c] = 13600 r + 1360 (:33-60); and the GEMV pattern
    W[r][c] = r + c, x[c] = c + 1  =>  y[r] = 136 r + 1360 (:70-76).  Every operand is an integer below 2048, exact in fp16."""
    r = np.arange(16, dtype=np.float32)
    a1 = 100.0 * r[:, None] + r[None, :]                      # [row][k]
    b1 = np.repeat((r + 1.0)[:, None], 16, axis=1)            # [k][col]
    c1 = np.repeat((13600.0 * r + 1360.0)[:, None], 16, axis=1)
    w2 = r[:, None] + r[None, :]                               # [row][c]
    x2 = (r + 1.0)[:, None]                                    # [c][1]
    y2 = (136.0 * r + 1360.0)[:, None]
    return (a1, b1, c1), (w2, x2, y2)
