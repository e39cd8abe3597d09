import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: test needs a CUDA device")
    config.addinivalue_line("markers", "device_scale_rounding: keep the library's default quantiser scale rounding "
                                       "(eager PyTorch on a CUDA device) instead of the CPU one")


@pytest.fixture(autouse=True)
def _scale_rounding_of_the_cpu_fixtures(request):
    """Most tests compare with the numpy oracle's default and with fixtures the reference produced on the CPU, which
    pin eager PyTorch's CPU scale rounding (max|x| / q_max); the library's default is the CUDA one.  Tests marked
    ``device_scale_rounding`` (fixtures the reference produced on a GPU) keep the default."""
    if "device_scale_rounding" in request.keywords:
        yield
        return
    from hyquant_b200 import decode_d_stage as dd
    old = dd.SCALE_MODE
    dd.SCALE_MODE = 0
    yield
    dd.SCALE_MODE = old
