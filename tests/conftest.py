"""Shared fixtures.  GPU tests are marked `gpu` and call through the C ABI;
everything else runs on a machine without a GPU."""
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def oracle():
    from oracle.loader import Oracle
    return Oracle()


@pytest.fixture(scope="session")
def reference():
    """The unmodified reference behind oracle/_ref, or skip when it was not built."""
    from oracle.loader import Reference, have_reference
    if not have_reference():
        pytest.skip("oracle/_ref is not built on this machine")
    return Reference()


@pytest.fixture(scope="session")
def lib():
    from cpu_ops_b200 import _capi, build
    build.build()
    return _capi.load()


@pytest.fixture(scope="session")
def lib_instrument():
    """The library built with -DCPUOPS_B200_INSTRUMENT: it alone exports the launch-policy
    probes (work order, tile-width choice).  Loaded beside the product library, never
    instead of it."""
    import ctypes
    from cpu_ops_b200 import build
    return ctypes.CDLL(str(build.build(instrument=True)))


@pytest.fixture(scope="session")
def gpu(lib):
    """Fails (does not skip) when a gpu-marked test runs without a usable device:
    a silent fallback must never look like a pass."""
    n = lib.cpuops_b200_device_count()
    assert n > 0, "gpu-marked test needs an sm_100 device; the library has no CPU fallback"
    return n
