import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def pkg():
    """The product package (ctypes binding of libesmm_b200.so); built on first use."""
    import __graft_entry__ as g
    if not os.path.exists(os.path.join(g.PKG_DIR, "libesmm_b200.so")):
        g.build()
    return g.load_package()


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.build()
    return oracle


@pytest.fixture(scope="session")
def cuda():
    """torch, used only for device buffers in the GPU tests."""
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    torch.cuda.set_device(0)
    return torch


@pytest.fixture
def tuning(pkg):
    """Sets the library's named tuning / test hooks (esmm_tuning_set) for one test and clears them afterwards."""
    L = pkg.lib()

    class Tuning:
        def __call__(self, name: str, value: int) -> None:
            assert L.esmm_tuning_set(name.encode(), int(value)) == 0, name

        def reset(self) -> None:
            L.esmm_tuning_reset()
    t = Tuning()
    t.reset()
    yield t
    t.reset()
