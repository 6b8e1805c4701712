import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `pytest -m gpu`)")


@pytest.fixture(autouse=True)
def _status_clean(request):
    """After every GPU test: raise if any kernel recorded a device-side error (bounded wait ran out, bounds check)."""
    yield
    if request.node.get_closest_marker("gpu"):
        import torch
        if torch.cuda.is_available():
            from aeris_gb_b200.ops import lib
            lib.check_status()


def rel_err(a, b):
    a, b = a.float(), b.float()
    return ((a - b).norm() / b.norm().clamp_min(1e-12)).item()


def free_port() -> int:
    import socket
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]
