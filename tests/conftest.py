import os
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle():
    from oracle import orc
    return orc.Oracle()


@pytest.fixture(scope="session")
def reference():
    from oracle import orc
    orc.build()
    if not orc.Reference.available():
        pytest.skip("oracle/_ref/libscn_ref.so not built (reference checkout absent)")
    return orc.Reference()
