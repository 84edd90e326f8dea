import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def lx():
    """The CUDA library through its C ABI. A missing library is an error, never a skip: there is no fallback."""
    from dromos_b200 import abi

    return abi.Library(abi.default_library_path())


@pytest.fixture(scope="session")
def ref():
    """The reference project's own CPU backend (oracle/_ref, built by oracle/Makefile), or a skip when it is absent."""
    from dromos_b200 import abi

    path = os.path.join(ROOT, "oracle", "_ref", "libdromos_cpu.so")
    if not os.path.exists(path):
        pytest.skip("oracle/_ref/libdromos_cpu.so not built (make -C oracle ref needs the reference checkout)")
    return abi.Library(path)
