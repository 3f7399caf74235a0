import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN_DIR = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


def golden(name):
    return np.load(os.path.join(GOLDEN_DIR, name + ".npz"))


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle

    oracle._lib()
    return oracle


@pytest.fixture(scope="session")
def ref_sim():
    """The reference simulator build (oracle/_ref); tests that need it skip where it was never built."""
    import oracle

    if not oracle.Ref.available():
        pytest.skip("oracle/_ref/libpto_ref.so not built (reference tree absent)")
    return oracle.Ref()
