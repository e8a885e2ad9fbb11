import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "diff-surfel-tracing_b200")
for p in (ROOT, PKG, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if p not in sys.path:
        sys.path.insert(0, p)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200 with `-m gpu`)")


@pytest.fixture(scope="session")
def oracle_mod():
    """The CPU oracle's ctypes front end; builds liboracle.so on first use when it is missing."""
    from oracle import build as obuild
    obuild.build_restatement()
    from oracle import oracle as orc
    return orc
