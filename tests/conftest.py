import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def port():
    from oracle import pyoracle
    return pyoracle.Oracle("port")


@pytest.fixture(scope="session")
def ref():
    """The reference's own operators; skipped where neither the reference
    checkout nor a prebuilt oracle/_ref is present."""
    from oracle import pyoracle
    if not pyoracle.Oracle.available("reference"):
        pytest.skip("oracle/_ref/libflref.so not available")
    return pyoracle.Oracle("reference")


@pytest.fixture(scope="session")
def checker():
    """The oracle GPU results are checked against: the reference's own code when
    its build is present, else the pinned port."""
    from oracle import pyoracle
    kind = "reference" if pyoracle.Oracle.available("reference") else "port"
    return pyoracle.Oracle(kind)


@pytest.fixture(scope="session")
def ctx():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from fast_llm_b200 import capi
    c = capi.Context(0)
    yield c
    c.close()
