import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (B200, sm_100a)")


def _has_gpu() -> bool:
    try:
        import torch

        return torch.cuda.is_available()
    except Exception:
        return False


def pytest_collection_modifyitems(config, items):
    if _has_gpu():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


@pytest.fixture(scope="session")
def oracle():
    from oracle import pyoracle

    pyoracle.build()
    return pyoracle.Oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own helpers compiled in place; None where oracle/_ref was not built."""
    from oracle import pyoracle

    pyoracle.build()
    if not pyoracle.Reference.available():
        return None
    return pyoracle.Reference()


@pytest.fixture(scope="session")
def capi():
    from nihilus_b200 import build

    build.build()
    from nihilus_b200 import capi as c

    return c


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    return np.load(os.path.join(ROOT, "tests", "golden", "q8_ref_vectors.npz"))
