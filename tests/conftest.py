import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) GPU; run with -m gpu")


@pytest.fixture(scope="session")
def oracle_lib():
    import oracle

    oracle.build()
    return oracle


@pytest.fixture(autouse=True)
def guard_bands_intact(request):
    """After every GPU test: no kernel wrote into the bands of 0xFF bytes around the device allocations of the
    contexts that are still open (the stand-in for a memory checker)."""
    yield
    if request.node.get_closest_marker("gpu") is None:
        return
    import moeflux_b200 as M

    for ctx in M.live_contexts():
        ctx.check_guards()
