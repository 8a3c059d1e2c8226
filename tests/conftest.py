import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
for p in (ROOT, os.path.join(ROOT, "oracle"), os.path.dirname(os.path.abspath(__file__))):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def golden_ops():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "ops_small.npz"))


@pytest.fixture(scope="session")
def golden_api():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "api_small.npz"))


@pytest.fixture(scope="session")
def oracle():
    """The plain-C restatement of the reference CPU algorithms (test infrastructure)."""
    import csr_oracle
    csr_oracle.build()
    return csr_oracle


@pytest.fixture(scope="session")
def reference_module():
    """The reference's own CPU operator module, if oracle/_ref has been built; else None."""
    import build_ref
    try:
        return build_ref.load()
    except ImportError:
        return None
