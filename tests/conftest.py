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


@pytest.fixture(scope="session")
def scn():
    """The product package (its directory name has a hyphen)."""
    import importlib
    return importlib.import_module("sparseconvnet-archived_b200")


@pytest.fixture(scope="session")
def abi(scn):
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    a = scn.abi
    a.lib()  # raises if libscn_b200.so is missing: GPU tests must never pass on a fallback
    assert a.lib().scn_device_supported() == 1, "libscn_b200.so is built for sm_100a only"
    return a
