import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def ctx():
    """One context for the whole GPU session (the C ABI is thread-affine, like the reference's worker)."""
    import pyre_b200 as pb

    c = pb.Ctx(0)
    yield c
    c.close()


def rel_err(y, ref):
    """max |y - ref| relative to the largest reference magnitude (scale of the computation)."""
    import numpy as np

    return float(np.abs(np.asarray(y, dtype=np.float64) - np.asarray(ref, dtype=np.float64)).max() / (np.abs(ref).max() + 1e-30))
