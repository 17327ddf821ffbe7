import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (run with -m gpu)")


@pytest.fixture(scope="session")
def qo():
    """The C oracle (built on demand)."""
    from oracle import qoracle
    qoracle.lib()
    return qoracle


@pytest.fixture(scope="session")
def ref():
    """The reference's own CPU kernels, or skip when the library is neither prebuilt nor buildable."""
    from oracle import ref as r
    if not r.available():
        try:
            r.build()
        except Exception:
            pass
    if not r.available():
        pytest.skip("oracle/_ref/libnncase_ref.so not available")
    return r


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no GPU")
    from nncase_b200.kernels import Context
    c = Context(0)
    yield c
    c.close()
