import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "torq-compiler_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def device():
    from torq_b200.runtime import Device
    d = Device(0)  # raises if the CUDA library or an sm_100 GPU is missing: no fallback
    yield d
    d.close()
