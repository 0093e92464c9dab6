import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a B200; run with -m gpu")


def rel_l2(got, want) -> float:
    got = np.asarray(got, np.float64).reshape(-1)
    want = np.asarray(want, np.float64).reshape(-1)
    den = np.linalg.norm(want)
    return float(np.linalg.norm(got - want) / (den if den > 0 else 1.0))


@pytest.fixture(scope="session")
def gpu():
    import ojas_engine_b200 as ob
    g = ob.B200Gpu(0)
    yield g
    g.close()
