import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import binding
    return binding.Oracle()


@pytest.fixture(scope="session")
def reflib():
    """The compiled reference, where oracle/_ref was built; else the test is skipped."""
    from oracle import binding
    if not binding.RefLib.available():
        pytest.skip("oracle/_ref/libgufo_ref.so was not built (no reference tree here)")
    return binding.RefLib()


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    here = os.path.join(ROOT, "tests", "golden")

    class Golden:
        def __init__(self):
            self._files = {}

        def __call__(self, name):
            if name not in self._files:
                self._files[name] = np.load(os.path.join(here, name + ".npz"))
            return self._files[name]

        def path(self, *parts):
            return os.path.join(here, *parts)

    return Golden()
