import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from tests import checkers
    return checkers.load_oracle()


@pytest.fixture(scope="session")
def refcpu():
    """minml's own CPU backend compiled from the reference sources (oracle/_ref); skipped when it was not built."""
    from tests import checkers
    ref = checkers.load_reference_cpu()
    if ref is None:
        pytest.skip("oracle/_ref/libminml_cpu_ref.so not built (needs the reference checkout)")
    return ref


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from minml_b200 import backend
    c = backend.Context(0)
    yield c
    c.close()
