import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tiny-dpcpp-nn_b200")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def tnn_lib():
    """The built C-ABI library; building is part of the fixture so a stale .so never hides a change."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("tnn_build", os.path.join(ROOT, "tiny-dpcpp-nn_b200", "build.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.build()
    from tiny_dpcpp_nn import _lib

    return _lib
