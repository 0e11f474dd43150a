import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
PACKAGE = ROOT / "triton-metal_b200"
for path in (str(ROOT), str(PACKAGE), str(ROOT / "tests")):
    if path not in sys.path:
        sys.path.insert(0, path)

LIBRARY = PACKAGE / "lib" / "libtmcuda.so"


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")
    if not LIBRARY.exists():
        # the product has no CPU fallback: without the built library nothing imports
        sys.path.insert(0, str(ROOT))
        import __graft_entry__
        __graft_entry__.build()


@pytest.fixture(scope="session")
def core():
    from triton_metal import _core
    return _core


@pytest.fixture()
def no_leaks(core):
    before = core.live_handle_count()
    yield
    assert core.live_handle_count() == before, "handles leaked"
