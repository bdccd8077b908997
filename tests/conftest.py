import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)
TESTS = os.path.dirname(os.path.abspath(__file__))
if TESTS not in sys.path:
    sys.path.insert(0, TESTS)


def pytest_addoption(parser):
    parser.addoption("--checked-lib", action="store_true", default=False,
                     help="run the suite on libesmm_b200_checked.so (the bounds-checked build) in the product library's place")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (runs on the B200 box)")


@pytest.fixture(scope="session")
def pkg(request):
    """The product package (ctypes binding of libesmm_b200.so); built on first use.  With --checked-lib the package binds
    the bounds-checked build instead, so that every GPU test doubles as a bounds check (esmm_device_status, which the
    tests read after their calls, reports a failed check)."""
    import __graft_entry__ as g
    if not os.path.exists(os.path.join(g.PKG_DIR, "libesmm_b200.so")):
        g.build()
    mod = g.load_package()
    if request.config.getoption("--checked-lib"):
        mod.LIB_PATH = mod.CHECKED_LIB_PATH
        assert mod.lib().esmm_checked_build() == 1
    return mod


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
