import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200); run with -m gpu")


@pytest.fixture(scope="session")
def restated():
    """The plain-C restatement of the path (oracle/d8_oracle.c), built on demand."""
    from oracle import pyoracle
    pyoracle.build(ref=False)
    return pyoracle.Restated()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU code (oracle/_ref/libd8ref.so); skipped where it was never built."""
    from oracle import pyoracle
    if not pyoracle.Reference.available():
        try:
            pyoracle.build(ref=True)
        except Exception:
            pass
    if not pyoracle.Reference.available():
        pytest.skip("oracle/_ref/libd8ref.so not built (reference tree absent)")
    return pyoracle.Reference()


@pytest.fixture(scope="session")
def ctx():
    """A d8k context on cuda:0.  The CUDA library is the product: a missing build is an error, not a skip."""
    import torch
    import deep8_b200
    assert torch.cuda.is_available(), "gpu tests need a CUDA device"
    c = deep8_b200.Context(0)
    yield c
    c.close()
