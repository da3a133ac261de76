import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (os.path.join(ROOT, "async-gpu_b200"), ROOT, os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu on the GPU box)")


@pytest.fixture(scope="session")
def reg():
    """One context for the whole GPU test session.  No skip: a missing library or GPU is a failure."""
    import b200nn

    r = b200nn.KernelRegistry.init_default()
    yield r
    r.close()
