"""Shared pytest set-up: markers, import path, and the oracle / library fixtures."""
import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 box)")


@pytest.fixture(scope="session")
def orc():
    """The CPU oracle (test infrastructure)."""
    from oracle import cpu_oracle
    cpu_oracle.build()
    return cpu_oracle


@pytest.fixture(scope="session")
def golden():
    import numpy as np
    d = os.path.join(ROOT, "tests", "golden")

    class G:
        quantize = np.load(os.path.join(d, "quantize.npz"))
        gemv = np.load(os.path.join(d, "gemv.npz"))
        pick = np.load(os.path.join(d, "pick.npz"))
        sample = np.load(os.path.join(d, "sample.npz"))

        @staticmethod
        def names(npz):
            return sorted({k.split(".")[0] for k in npz.files})

    return G
