import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    path = os.path.join(ROOT, "tests", "golden", "reference_vectors.npz")
    return np.load(path)


@pytest.fixture(autouse=True, scope="session")
def _poison_outputs():
    """Every output tensor the binding allocates during the tests starts as NaN, so an element a kernel forgot
    to write cannot inherit a correct value left in that memory by an earlier test."""
    try:
        from flex_attention_tpu_b200 import _binding
    except ImportError:
        yield
        return
    old, _binding.POISON_OUTPUTS = _binding.POISON_OUTPUTS, True
    yield
    _binding.POISON_OUTPUTS = old
