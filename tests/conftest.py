import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


def reference_package():
    """Import the upstream package for differential tests; None when it is not on this machine."""
    for cand in (os.path.join(ROOT, "baseline", "_ref"), os.environ.get("EPLB_REFERENCE_DIR", "")):
        if os.path.isdir(os.path.join(cand, "eplb")):
            if cand not in sys.path:
                sys.path.append(cand)
            try:
                import eplb  # noqa: F401

                return eplb
            except Exception:
                return None
    return None


@pytest.fixture(scope="session")
def ref_eplb():
    mod = reference_package()
    if mod is None:
        pytest.skip("reference package not available")
    return mod
