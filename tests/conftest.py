import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200 (sm_100) device")


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    return np.load(os.path.join(ROOT, "tests", "golden", "legacy_reference.npz"))


@pytest.fixture(scope="session")
def oracle_mod():
    import oracle
    oracle.lib()  # builds the restatement on first use
    return oracle


@pytest.fixture(scope="session")
def built_lib():
    from patina_b200 import build
    build.build_library()
    from patina_b200 import lib
    return lib.load()
