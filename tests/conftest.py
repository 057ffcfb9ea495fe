import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle as orc  # oracle/oracle.py

    orc.lib()
    return orc


@pytest.fixture(scope="session")
def hm():
    """The product library through its ctypes binding."""
    import homura_b200

    homura_b200.load_library()
    return homura_b200
