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
    from oracle import pelica_oracle as po

    po.build()
    return po


@pytest.fixture(scope="session")
def ctx():
    """The CUDA context of the product library. No fallback: without the built
    library or a GPU this fails the test instead of skipping it."""
    import pelica_b200 as pb

    c = pb.Context(0)
    yield c
    c.close()
