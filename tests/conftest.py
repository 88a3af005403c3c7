import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

GOLDEN = os.path.join(ROOT, "tests", "golden")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import load_oracle
    return load_oracle()


@pytest.fixture(scope="session")
def reference():
    """The reference's own CPU library, if oracle/_ref was built where the checkout exists."""
    from oracle import load_reference
    return load_reference()


@pytest.fixture(scope="session")
def golden():
    import numpy as np

    class G:
        walks = np.load(os.path.join(GOLDEN, "walks.npz"))
        mlp = np.load(os.path.join(GOLDEN, "mlp.npz"))
        adamw = np.load(os.path.join(GOLDEN, "adamw.npz"))
        plan = np.load(os.path.join(GOLDEN, "plan.npz"))
    return G
