"""B200-native forward path for spatially-sparse CNNs (drop-in for the forward path of
btgraham/SparseConvNet-archived).

The directory name contains a hyphen, so import it with
    importlib.import_module("sparseconvnet-archived_b200")
`abi` binds the C ABI of libscn_b200.so (include/scn_b200.h); `net` binds the harness entry
points of libscn_b200_host.so (include/scn_b200_net.h), behind which live the C++ classes
that keep the reference's names.  There is no CPU fallback: every call fails loudly if the
CUDA libraries are missing.
"""
import importlib
import os

PKG_DIR = os.path.dirname(os.path.abspath(__file__))
KERNEL_LIB = os.path.join(PKG_DIR, "libscn_b200.so")
HOST_LIB = os.path.join(PKG_DIR, "libscn_b200_host.so")


def build(verbose=False):
    """Compile both shared libraries in-tree for sm_100a (nvcc cross-compiles without a GPU)."""
    import subprocess
    cmd = ["make", "-C", os.path.join(PKG_DIR, "csrc"), "-j4", "all"]
    res = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building libscn_b200 failed")


def __getattr__(name):
    if name in ("abi", "net", "synth", "shard"):
        return importlib.import_module(__name__ + "." + name)
    raise AttributeError(name)
