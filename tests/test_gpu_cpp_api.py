"""Builds and runs tests/cpp/test_host_api.cpp: a C++ program written against the reference's
class names (DeepCNet, SparseConvNet, layer preprocess()/forwards(), gridRules, vectorCUDA,
BatchProducer) linked against the two in-tree libraries."""
import os
import subprocess

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PKG = os.path.join(ROOT, "sparseconvnet-archived_b200")
SRC = os.path.join(ROOT, "tests", "cpp", "test_host_api.cpp")
EXE = os.path.join(ROOT, "tests", "cpp", "test_host_api")


def build_exe():
    cmd = ["g++", "-std=c++17", "-O1", "-o", EXE, SRC, "-I" + os.path.join(PKG, "csrc", "host"), "-I" + os.path.join(ROOT, "include"),
           "-I/usr/local/cuda/include", "-L" + PKG, "-lscn_b200_host", "-lscn_b200", "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + PKG, "-Wl,-rpath,/usr/local/cuda/lib64", "-pthread"]
    subprocess.run(cmd, check=True)


def test_cpp_program_compiles(scn):
    """The reference-style program compiles and links against the headers and libraries (no GPU)."""
    if not (os.path.exists(scn.KERNEL_LIB) and os.path.exists(scn.HOST_LIB)):
        scn.build()
    build_exe()
    assert os.path.exists(EXE)


def test_dataset_helpers_program_runs_on_the_host(scn):
    """tests/cpp/test_dataset_helpers.cpp: the data set helpers need no GPU."""
    if not (os.path.exists(scn.KERNEL_LIB) and os.path.exists(scn.HOST_LIB)):
        scn.build()
    src = os.path.join(ROOT, "tests", "cpp", "test_dataset_helpers.cpp")
    exe = os.path.join(ROOT, "tests", "cpp", "test_dataset_helpers")
    cmd = ["g++", "-std=c++17", "-O1", "-o", exe, src, "-I" + os.path.join(PKG, "csrc", "host"), "-I" + os.path.join(ROOT, "include"),
           "-I/usr/local/cuda/include", "-L" + PKG, "-lscn_b200_host", "-lscn_b200", "-L/usr/local/cuda/lib64", "-lcudart",
           "-Wl,-rpath," + PKG, "-Wl,-rpath,/usr/local/cuda/lib64", "-pthread"]
    subprocess.run(cmd, check=True)
    res = subprocess.run([exe], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=60)
    assert res.returncode == 0 and "ALL OK" in res.stdout, res.stdout[-2000:]


@pytest.mark.gpu
def test_cpp_program_runs(abi):
    build_exe()
    res = subprocess.run([EXE], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, timeout=300)
    assert res.returncode == 0, res.stdout[-3000:]
    assert "ALL OK" in res.stdout
