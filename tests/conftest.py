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


# Largest |error| seen per kind of comparison (relative to the largest reference value), written at the end
# of the session so that the measured margins can be quoted next to the stated tolerances.
_ERRORS = {}


def record_error(what: str, err: float, ref: float):
    cur = _ERRORS.get(what)
    if cur is None or err / ref > cur[0] / cur[1]:
        _ERRORS[what] = (err, ref)


def pytest_sessionfinish(session, exitstatus):
    if not _ERRORS:
        return
    out = os.environ.get("HM_ERROR_REPORT")
    lines = [f"{k}: max-abs {e:.3e} at reference scale {r:.3e} (relative {e / r:.2e})" for k, (e, r) in sorted(_ERRORS.items())]
    print("\n[measured errors]\n" + "\n".join(lines))
    if out:
        with open(out, "w") as f:
            f.write("\n".join(lines) + "\n")
