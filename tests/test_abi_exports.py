"""CPU checks: both shared libraries load and export every function their headers declare,
and the product never touches the oracle."""
import ctypes
import os
import re
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sparseconvnet-archived_b200")


def declared(header):
    text = open(os.path.join(ROOT, "include", header)).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(scn_[a-zA-Z0-9_]+)\s*\(", text)))


@pytest.fixture(scope="module")
def built(scn):
    if not (os.path.exists(scn.KERNEL_LIB) and os.path.exists(scn.HOST_LIB)):
        scn.build()
    return scn


@pytest.mark.parametrize("header,libattr", [("scn_b200.h", "KERNEL_LIB"), ("scn_b200_net.h", "HOST_LIB")])
def test_every_declared_symbol_is_exported(built, header, libattr):
    ctypes.CDLL(built.KERNEL_LIB, mode=ctypes.RTLD_GLOBAL)
    lib = ctypes.CDLL(getattr(built, libattr))
    names = declared(header)
    assert len(names) >= 10
    for n in names:
        assert hasattr(lib, n), "%s is declared in include/%s but not exported" % (n, header)


def test_python_bindings_cover_the_headers(built):
    assert sorted(built.abi.EXPORTS) == declared("scn_b200.h")
    assert sorted(built.net.EXPORTS) == declared("scn_b200_net.h")


def test_argument_checks_need_no_gpu(built):
    """Status codes and messages work without a device (no compute call is made)."""
    L = built.abi.lib()
    assert L.scn_status_string(0) == b"ok"
    R = built.abi.regions(0, 2, 9, 6, 3, 1, 1)  # nIn != size + (nOut-1)*stride
    assert L.scn_regions_cells(ctypes.byref(R)) == -1
    assert b"nIn" in L.scn_last_error()
    R = built.abi.regions(1, 3, 47, 46, 2, 1, 2)
    assert L.scn_regions_cells(ctypes.byref(R)) == 4  # tetrahedral filter of side 2
    assert L.scn_rules_workspace_bytes(ctypes.byref(R), 4, 1000) > 0


def test_product_does_not_reach_into_the_oracle():
    hits = subprocess.run(["grep", "-rIl", "-E", r"oracle|orc_|_ref", PKG, "--include=*.py", "--include=*.cu",
                           "--include=*.cuh", "--include=*.cpp", "--include=*.h"], stdout=subprocess.PIPE, text=True).stdout
    assert hits.strip() == "", "product files mention the oracle:\n" + hits
