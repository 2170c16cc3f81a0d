"""Pins the oracle's rule construction and scalar helpers to the reference's own code
(Regions.cu, utilities.cu compiled unchanged into oracle/_ref)."""
import numpy as np
import pytest

from gridgen import random_grids


def same(a, b):
    assert a["n_sites"] == b["n_sites"]
    for k in ("rules", "out_keys", "out_rows", "out_off", "out_bg"):
        np.testing.assert_array_equal(a[k], b[k], err_msg=k)


def test_scalar_helpers(oracle, reference):
    for b in range(1, 8):
        for e in range(0, 6):
            assert oracle.lib.orc_ipow(b, e) == reference.lib.ref_ipow(b, e)
    for s in range(1, 12):
        for d in range(1, 5):
            assert oracle.lib.orc_triangleSize(s, d) == reference.lib.ref_triangleSize(s, d)
    for a in range(0, 700, 7):
        assert oracle.lib.orc_intRound(a, 32) == reference.lib.ref_intRound(a, 32)


def test_top_indices(oracle, reference):
    rng = np.random.default_rng(3)
    for n in (1, 2, 5, 10, 101):
        for k in (1, 2, 5):
            if k > n:
                continue
            for _ in range(20):
                v = rng.standard_normal(n).astype(np.float32)
                if rng.random() < 0.3:
                    v = np.round(v)  # ties
                np.testing.assert_array_equal(oracle.top_indices(v, k), reference.top_indices(v, k))


# (dim, nOut, size, stride, minActive)
SQUARE = [
    (1, 9, 3, 1, 1), (1, 5, 2, 2, 1), (1, 6, 3, 2, 1),
    (2, 6, 3, 1, 1), (2, 7, 2, 1, 1), (2, 5, 2, 2, 1), (2, 4, 3, 2, 1), (2, 3, 3, 3, 1), (2, 1, 2, 1, 1),
    (3, 5, 3, 1, 1), (3, 6, 2, 1, 1), (3, 4, 2, 2, 1), (3, 3, 3, 2, 1),
    (1, 6, 3, 1, 2), (2, 6, 3, 1, 2), (2, 6, 2, 1, 3), (2, 5, 2, 2, 2), (3, 5, 2, 1, 2), (3, 4, 3, 1, 4),
    (4, 3, 2, 1, 2), (4, 2, 2, 2, 3),
    (2, 7, 3, 1, -1),
]


@pytest.mark.parametrize("dim,nOut,size,stride,minActive", SQUARE)
def test_square_rules(oracle, reference, dim, nOut, size, stride, minActive):
    nIn = size + (nOut - 1) * stride
    rng = np.random.default_rng(1000 * dim + 10 * nOut + size + stride)
    for density in (0.0, 0.03, 0.3, 0.8, 1.0):
        for with_bg in (True, False):
            if density < 1.0 and not with_bg and minActive != 1:
                pass  # backgroundCol -1 with missing cells is legal: cells hold -1
            g = random_grids(rng, 3, dim, nIn, density, with_bg=with_bg, first_row=int(rng.integers(0, 5)))
            a = oracle.grid_rules(0, dim, nIn, nOut, size, stride, minActive, *g)
            b = reference.grid_rules(0, dim, nIn, nOut, size, stride, minActive, *g)
            same(a, b)


TRI = [
    (2, 6, 2, 1, 1), (2, 5, 3, 1, 1), (2, 4, 2, 2, 1), (2, 3, 3, 2, 1),
    (3, 5, 2, 1, 1), (3, 4, 3, 1, 1), (3, 4, 2, 2, 1), (4, 3, 2, 1, 1), (4, 2, 2, 2, 1),
    (1, 5, 2, 1, 2), (2, 6, 2, 1, 2), (2, 5, 3, 1, 3), (3, 5, 2, 1, 2), (3, 4, 3, 1, 2), (3, 3, 2, 2, 2), (4, 3, 2, 1, 2),
]


@pytest.mark.parametrize("dim,nOut,size,stride,minActive", TRI)
def test_triangular_rules(oracle, reference, dim, nOut, size, stride, minActive):
    nIn = size + (nOut - 1) * stride
    rng = np.random.default_rng(77 + 1000 * dim + 10 * nOut + size + stride)
    for density in (0.0, 0.05, 0.3, 0.8, 1.0):
        for with_bg in (True, False):
            g = random_grids(rng, 3, dim, nIn, density, triangular=True, with_bg=with_bg)
            a = oracle.grid_rules(1, dim, nIn, nOut, size, stride, minActive, *g)
            b = reference.grid_rules(1, dim, nIn, nOut, size, stride, minActive, *g)
            same(a, b)


def test_chain_matches_reference(oracle, reference):
    """conv3 -> MP2 -> conv2 -> MP2 chained through each library's own outputs."""
    rng = np.random.default_rng(5)
    for dim, S in ((2, 24), (3, 12)):
        g = random_grids(rng, 4, dim, S, [0.02, 0.2, 0.6, 1.0])
        cur_o, cur_r = g, g
        n = S
        for size, stride in ((3, 1), (2, 2), (2, 1), (2, 2)):
            nOut = (n - size) // stride + 1
            a = oracle.grid_rules(0, dim, n, nOut, size, stride, 1, *cur_o)
            b = reference.grid_rules(0, dim, n, nOut, size, stride, 1, *cur_r)
            same(a, b)
            cur_o = (a["out_keys"], a["out_rows"], a["out_off"], a["out_bg"])
            cur_r = (b["out_keys"], b["out_rows"], b["out_off"], b["out_bg"])
            n = nOut


# Fractional max-pooling (MaxPoolingLayer.cu:157-407): (kind, dim, nOut, shrink); poolSize 2 as in the
# named FMP architectures; nIn as the layers' calculateInputSpatialSize derives it.
FMP = [(k, d, n, s) for k in range(4) for d, n, s in [(1, 7, 1.414), (2, 5, 1.26), (2, 6, 1.5), (2, 9, 1.7), (3, 4, 1.414), (3, 5, 1.26)]]
# 4-D only for the non-overlapping kinds: the reference's 4-D gridRulesOverlappingNoMin starts axis 0 at
# outputL(0, i1) (Regions.cu:613), which indexes outside its rule rows
FMP += [(1, 4, 3, 1.5), (3, 4, 3, 1.5), (1, 2, 10, 2.0)]


def fmp_nin(nOut, shrink):
    nIn = int(nOut * np.float32(shrink) + 0.5)
    return nIn + 1 if nIn == nOut else nIn


@pytest.mark.parametrize("kind,dim,nOut,shrink", FMP)
def test_fmp_ticks_and_rules(oracle, reference, kind, dim, nOut, shrink):
    """The tick tables (the reference's RNG draw by draw) and both FMP rule builders."""
    nIn = fmp_nin(nOut, shrink)
    rng = np.random.default_rng(31 * kind + 7 * dim + nOut)
    for density in (0.0, 0.1, 0.5, 1.0):
        for with_bg in (True, False):
            seed = int(rng.integers(1, 2 ** 31))
            g = random_grids(rng, 4, dim, nIn, density, with_bg=with_bg, first_row=int(rng.integers(0, 5)))
            ref, ticks = reference.fmp_rules(kind, dim, nIn, nOut, 2, seed, *g)
            np.testing.assert_array_equal(oracle.fmp_ticks(kind, dim, nIn, nOut, 2, seed, 4), ticks)
            same(oracle.fmp_rules(dim, nIn, nOut, 2, kind in (0, 2), ticks, *g), ref)
