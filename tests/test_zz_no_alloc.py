"""scn_rules_build_static: rule construction for hosts that are not allowed to allocate GPU
memory (a framework owns the device's memory, or the caller sits on a path that must never
enter cudaMalloc).  Its scratch is a fixed array inside the library, so this test calls it
through the C ABI twice in a row -- the second call finds the first call's leftovers in the
array -- and requires exactly the rulebooks the ordinary entry point produces (integers:
bit-exact).  The file name sorts last on purpose: with `pytest -x` every other test has run
before this one."""
import numpy as np
import pytest
import torch

from gridgen import random_grids
from test_gpu_rules import to_dev_grid

pytestmark = pytest.mark.gpu


def _both(abi, lattice, dim, nOut, size, stride, min_active, g, reuse=None):
    nIn = size + (nOut - 1) * stride
    dk, doff, dbg, _ = to_dev_grid(*g)
    R = abi.regions(lattice, dim, nIn, nOut, size, stride, min_active)
    cap = dk.numel() * ((size + stride - 1) // stride) ** dim + len(g[3]) + 8
    ref = abi.rules_build(R, dk, doff, dbg, cap)            # caller-owned workspace
    got = abi.rules_build_static(R, dk, doff, dbg, cap, out=reuse)  # the library's fixed array
    torch.cuda.synchronize()
    r, s = ref["result"].cpu().numpy(), got["result"].cpu().numpy()
    np.testing.assert_array_equal(s, r)
    assert r[2] == 0
    rows, sd = int(r[0]), ref["sd"]
    np.testing.assert_array_equal(got["rules"].cpu().numpy()[: rows * sd], ref["rules"].cpu().numpy()[: rows * sd])
    np.testing.assert_array_equal(got["out_keys"].cpu().numpy()[:rows], ref["out_keys"].cpu().numpy()[:rows])
    np.testing.assert_array_equal(got["out_off"].cpu().numpy(), ref["out_off"].cpu().numpy())
    np.testing.assert_array_equal(got["out_bg"].cpu().numpy(), ref["out_bg"].cpu().numpy())
    return rows, got


def test_two_calls_in_a_row_match_the_allocating_entry_point(abi):
    rng = np.random.default_rng(123)
    # first a large, dense build, so the array is full of stale bits, counts and flags ...
    g1 = random_grids(rng, 8, 2, 24, 0.6)
    rows1, _ = _both(abi, 0, 2, 22, 3, 1, 1, g1)
    # ... then a sparser one of another geometry straight after it, then the first again
    g2 = random_grids(rng, 5, 3, 8, 0.05)
    rows2, _ = _both(abi, 0, 3, 4, 2, 2, 1, g2)
    g3 = random_grids(rng, 6, 3, 7, 0.3, triangular=True)
    rows3, _ = _both(abi, 1, 3, 6, 2, 1, 2, g3)
    rows1b, _ = _both(abi, 0, 2, 22, 3, 1, 1, g1)
    assert rows1 == rows1b and rows1 > 0 and rows2 > 0 and rows3 > 0


def test_the_call_creates_no_device_memory(abi):
    """With the outputs handed in, the call leaves torch's allocator untouched and the device's
    free memory unchanged (a cudaMalloc inside the library would show in cudaMemGetInfo)."""
    rng = np.random.default_rng(5)
    g = random_grids(rng, 4, 2, 12, 0.4)
    _, out = _both(abi, 0, 2, 10, 3, 1, 1, g)  # first call: address look-up done, outputs exist
    dk, doff, dbg, _ = to_dev_grid(*g)
    R = abi.regions(0, 2, 12, 10, 3, 1, 1)
    unchanged = False
    for _ in range(3):  # free memory is device-wide: allow for an unrelated change and look again
        torch.cuda.synchronize()
        free0, _ = torch.cuda.mem_get_info()
        stats0 = torch.cuda.memory_stats()["allocation.all.allocated"]
        abi.rules_build_static(R, dk, doff, dbg, out["out_keys"].numel(), out=out)
        torch.cuda.synchronize()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == stats0
        unchanged = unchanged or torch.cuda.mem_get_info()[0] == free0
    assert unchanged


def test_sizes_beyond_the_fixed_array_are_refused(abi):
    limit = abi.lib().scn_rules_static_scratch_bytes()
    assert limit == 16 << 20
    z = torch.zeros(8, dtype=torch.int32, device="cuda")
    R = abi.regions(0, 3, 66, 64, 3, 1, 1)  # 66^3 cells x 300 samples: bitmap alone is > 16 MiB
    with pytest.raises(abi.ScnError) as e:
        abi.rules_build_static(R, z, torch.zeros(301, dtype=torch.int32, device="cuda"), torch.zeros(300, dtype=torch.int32, device="cuda"), 16)
    assert "workspace" in str(e.value) and str(limit) in str(e.value)
