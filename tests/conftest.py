"""pytest configuration: registers the `gpu` marker and puts the repo's two
Python entry points (the ctypes binding and the oracle wrapper) on sys.path."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "go-metal_b200", "python"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")
    config.addinivalue_line("markers", "slow: a full-size, full-length configuration (minutes); deselect with -m 'gpu and not slow'")


@pytest.fixture(scope="session")
def gm():
    """The ctypes binding; building the library first if it is missing."""
    lib_path = os.path.join(ROOT, "go-metal_b200", "lib", "libgometal_cuda.so")
    if not os.path.exists(lib_path):
        import importlib.util
        spec = importlib.util.spec_from_file_location("gm_build", os.path.join(ROOT, "go-metal_b200", "build.py"))
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        mod.build()
    import gometal_cuda
    return gometal_cuda


@pytest.fixture(scope="session")
def dev(gm):
    """One device handle for the whole GPU session (fails loudly without a GPU)."""
    d = gm.Device()
    yield d
    d.close()


@pytest.fixture(scope="session")
def oracle():
    from oracle import oracle as O
    O.lib()
    return O
