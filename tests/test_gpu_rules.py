"""GPU parity (bit-exact): scn_rules_build / scn_terminal_rules_build through the C ABI
against the oracle's rule construction on the same seeded grids."""
import numpy as np
import pytest
import torch

from gridgen import random_grids

pytestmark = pytest.mark.gpu


def to_dev_grid(keys, rows, off, bg):
    """Flat (keys, rows) protocol -> device keys[row] / off / bg (rows are contiguous per
    sample, background row included)."""
    first = int(min([r for r in rows.tolist()] + [b for b in bg.tolist() if b >= 0] + [10 ** 9]))
    if first == 10 ** 9:
        first = 0
    n_rows = len(rows) + int((bg >= 0).sum())
    dk = np.full(n_rows, -1, np.int32)
    doff = np.zeros(len(bg) + 1, np.int32)
    row_lo = first
    for b in range(len(bg)):
        doff[b] = row_lo - first
        cnt = off[b + 1] - off[b] + (1 if bg[b] >= 0 else 0)
        row_lo += cnt
    doff[len(bg)] = row_lo - first
    dk[rows - first] = keys
    dbg = np.where(bg >= 0, bg - first, -1).astype(np.int32)
    return (torch.from_numpy(dk).cuda(), torch.from_numpy(doff).cuda(), torch.from_numpy(dbg).cuda(), first)


def run_gpu(abi, lattice, dim, nIn, nOut, size, stride, minActive, g, capacity=None):
    dk, doff, dbg, first = to_dev_grid(*g)
    assert first == 0
    R = abi.regions(lattice, dim, nIn, nOut, size, stride, minActive)
    T = ((size + stride - 1) // stride) ** dim
    cap = capacity if capacity is not None else dk.numel() * max(T, 1) + len(g[3]) + 8
    out = abi.rules_build(R, dk, doff, dbg, cap)
    torch.cuda.synchronize()
    res = out["result"].cpu().numpy()
    return out, res


def compare(out, res, ref):
    rows, sites, err, _ = (int(v) for v in res)
    assert err == 0
    assert rows == ref["n_sites"]
    sd = out["sd"]
    np.testing.assert_array_equal(out["rules"].cpu().numpy()[: rows * sd], ref["rules"])
    np.testing.assert_array_equal(out["out_bg"].cpu().numpy(), ref["out_bg"])
    gk = out["out_keys"].cpu().numpy()[:rows]
    goff = out["out_off"].cpu().numpy()
    # rebuild the (key, row) listing per sample in ascending key order
    keys, rws = [], []
    for b in range(len(ref["out_bg"])):
        lo, hi = goff[b], goff[b + 1]
        k = gk[lo:hi]
        r = np.arange(lo, hi)
        m = k >= 0
        order = np.argsort(k[m], kind="stable")
        keys.append(k[m][order]); rws.append(r[m][order])
        assert (~m).sum() == (1 if ref["out_bg"][b] >= 0 else 0)
        if ref["out_bg"][b] >= 0:
            assert r[~m][0] == ref["out_bg"][b]
        assert len(k[m]) == ref["out_off"][b + 1] - ref["out_off"][b]
    np.testing.assert_array_equal(np.concatenate(keys) if keys else np.zeros(0), ref["out_keys"])
    np.testing.assert_array_equal(np.concatenate(rws) if rws else np.zeros(0), ref["out_rows"])
    assert sites == len(ref["out_keys"])


SQUARE = [
    (1, 9, 3, 1, 1), (1, 5, 2, 2, 1), (1, 6, 3, 2, 1),
    (2, 6, 3, 1, 1), (2, 7, 2, 1, 1), (2, 5, 2, 2, 1), (2, 4, 3, 2, 1), (2, 3, 3, 3, 1), (2, 1, 2, 1, 1),
    (3, 5, 3, 1, 1), (3, 6, 2, 1, 1), (3, 4, 2, 2, 1), (3, 3, 3, 2, 1), (4, 3, 2, 1, 1), (4, 2, 3, 1, 1),
    (1, 6, 3, 1, 2), (2, 6, 3, 1, 2), (2, 6, 2, 1, 3), (2, 5, 2, 2, 2), (3, 5, 2, 1, 2), (3, 4, 3, 1, 4),
    (4, 3, 2, 1, 2), (4, 2, 2, 2, 3),
    (2, 7, 3, 1, -1), (3, 4, 3, 1, -1),
]


@pytest.mark.parametrize("dim,nOut,size,stride,minActive", SQUARE)
def test_square_rules(abi, oracle, dim, nOut, size, stride, minActive):
    nIn = size + (nOut - 1) * stride
    rng = np.random.default_rng(1000 * dim + 10 * nOut + size + stride)
    for density in (0.0, 0.03, 0.3, 0.8, 1.0):
        for with_bg in (True, False):
            g = random_grids(rng, 5, dim, nIn, density, with_bg=with_bg)
            ref = oracle.grid_rules(0, dim, nIn, nOut, size, stride, minActive, *g)
            out, res = run_gpu(abi, 0, dim, nIn, nOut, size, stride, minActive, g)
            compare(out, res, ref)


TRI = [
    (2, 6, 2, 1, 1), (2, 5, 3, 1, 1), (2, 4, 2, 2, 1), (2, 3, 3, 2, 1),
    (3, 5, 2, 1, 1), (3, 4, 3, 1, 1), (3, 4, 2, 2, 1), (4, 3, 2, 1, 1), (4, 2, 2, 2, 1),
    (1, 5, 2, 1, 2), (2, 6, 2, 1, 2), (2, 5, 3, 1, 3), (3, 5, 2, 1, 2), (3, 4, 3, 1, 2), (3, 3, 2, 2, 2), (4, 3, 2, 1, 2),
]


@pytest.mark.parametrize("dim,nOut,size,stride,minActive", TRI)
def test_triangular_rules(abi, oracle, dim, nOut, size, stride, minActive):
    nIn = size + (nOut - 1) * stride
    rng = np.random.default_rng(77 + 1000 * dim + 10 * nOut + size + stride)
    for density in (0.0, 0.05, 0.3, 0.8, 1.0):
        for with_bg in (True, False):
            g = random_grids(rng, 5, dim, nIn, density, triangular=True, with_bg=with_bg)
            ref = oracle.grid_rules(1, dim, nIn, nOut, size, stride, minActive, *g)
            out, res = run_gpu(abi, 1, dim, nIn, nOut, size, stride, minActive, g)
            compare(out, res, ref)


def test_larger_batches_and_ragged(abi, oracle):
    """Config-shaped geometry: ragged site counts, empty samples, many samples."""
    rng = np.random.default_rng(11)
    cases = [(2, 96, 3, 1, 64, [0.0, 0.11, 0.5]), (2, 94, 2, 2, 64, [0.02, 0.3]),
             (3, 48, 3, 1, 6, [0.0, 0.01, 0.05]), (3, 46, 2, 2, 6, [0.03, 0.2]), (3, 23, 2, 1, 9, [0.1, 0.6, 1.0])]
    for dim, nIn, size, stride, batch, dens in cases:
        nOut = (nIn - size) // stride + 1
        g = random_grids(rng, batch, dim, nIn, dens)
        ref = oracle.grid_rules(0, dim, nIn, nOut, size, stride, 1, *g)
        out, res = run_gpu(abi, 0, dim, nIn, nOut, size, stride, 1, g)
        compare(out, res, ref)


def test_chain_on_device(abi, oracle):
    """Feed each layer's device outputs straight into the next build (no host round trip of
    the grids), as the network driver does."""
    rng = np.random.default_rng(5)
    for dim, S in ((2, 24), (3, 12)):
        g = random_grids(rng, 7, dim, S, [0.02, 0.2, 0.6, 1.0, 0.0])
        cur = g
        dk, doff, dbg, _ = to_dev_grid(*g)
        n = S
        for size, stride in ((3, 1), (2, 2), (2, 1), (2, 2)):
            nOut = (n - size) // stride + 1
            ref = oracle.grid_rules(0, dim, n, nOut, size, stride, 1, *cur)
            R = abi.regions(0, dim, n, nOut, size, stride, 1)
            cap = dk.numel() * ((size + stride - 1) // stride) ** dim + 16
            out = abi.rules_build(R, dk, doff, dbg, cap)
            torch.cuda.synchronize()
            res = out["result"].cpu().numpy()
            compare(out, res, ref)
            rows = int(res[0])
            dk, doff, dbg = out["out_keys"][:rows].contiguous(), out["out_off"], out["out_bg"]
            cur = (ref["out_keys"], ref["out_rows"], ref["out_off"], ref["out_bg"])
            n = nOut


def test_capacity_and_bad_keys_are_reported(abi):
    rng = np.random.default_rng(2)
    g = random_grids(rng, 2, 2, 8, 0.5)
    out, res = run_gpu(abi, 0, 2, 8, 6, 3, 1, 1, g, capacity=3)
    assert res[2] & abi.DEV_ERR_CAPACITY
    dk, doff, dbg, _ = to_dev_grid(*g)
    dk2 = dk.clone()
    site = int((dk2 >= 0).nonzero()[0])
    dk2[site] = 8 * 8 + 5  # outside the grid
    out = abi.rules_build(abi.regions(0, 2, 8, 6, 3, 1, 1), dk2, doff, dbg, 200)
    torch.cuda.synchronize()
    assert int(out["result"][2]) & abi.DEV_ERR_KEY
    dk3 = dk.clone()
    sites = (dk3 >= 0).nonzero().flatten()
    same = [int(s) for s in sites if int(s) < int(doff[1])][:2]
    dk3[same[1]] = dk3[same[0]]
    out = abi.rules_build(abi.regions(0, 2, 8, 6, 3, 1, 1), dk3, doff, dbg, 200)
    torch.cuda.synchronize()
    assert int(out["result"][2]) & abi.DEV_ERR_DUPLICATE


def test_invalid_geometry_is_rejected(abi):
    z = torch.zeros(4, dtype=torch.int32, device="cuda")
    with pytest.raises(abi.ScnError):
        abi.rules_build(abi.regions(0, 2, 9, 6, 3, 1, 1), z, z[:2], z[:1], 10)  # nIn != size+(nOut-1)*stride
    with pytest.raises(abi.ScnError):
        abi.rules_build(abi.regions(0, 5, 8, 6, 3, 1, 1), z, z[:2], z[:1], 10)  # dim 5
    with pytest.raises(abi.ScnError):
        abi.rules_build(abi.regions(1, 2, 8, 6, 3, 1, -1), z, z[:2], z[:1], 10)  # valid on a triangular lattice


def test_terminal_rules(abi, oracle):
    rng = np.random.default_rng(9)
    for dim, S in ((2, 3), (3, 2), (3, 3)):
        for dens in ([0.0, 0.5, 1.0], [0.0], [0.3]):
            g = random_grids(rng, 6, dim, S, dens)
            ref = oracle.grid_rules(2, dim, S, 1, 1, 1, 1, *g)
            dk, doff, dbg, _ = to_dev_grid(*g)
            width = len(ref["rules"]) // 6
            out = abi.terminal_rules_build(dim, S, dk, doff, dbg, width)
            torch.cuda.synchronize()
            assert int(out["result"][2]) == 0 and int(out["result"][0]) == 6
            np.testing.assert_array_equal(out["rules"].cpu().numpy(), ref["rules"])
            np.testing.assert_array_equal(out["out_off"].cpu().numpy(), np.arange(7))
            np.testing.assert_array_equal(out["out_bg"].cpu().numpy(), ref["out_bg"])
            np.testing.assert_array_equal(out["out_keys"].cpu().numpy(), np.zeros(6))


CHAINS = [
    # (lattice, dim, S, [(size, stride, minActive), ...])
    (0, 2, 24, [(3, 1, 1), (2, 2, 1), (2, 1, 1), (2, 2, 1), (2, 1, 1)]),
    (0, 2, 26, [(3, 1, -1), (3, 1, 2), (2, 2, 1), (3, 2, 1)]),
    (0, 3, 12, [(3, 1, 1), (2, 2, 1), (2, 1, 2), (2, 2, 1)]),
    (1, 3, 11, [(2, 1, 2), (2, 2, 1), (2, 1, 1), (2, 2, 1)]),
    (1, 2, 14, [(3, 1, 1), (2, 2, 1), (2, 1, 3)]),
    (0, 1, 21, [(3, 1, 1), (3, 2, 1), (2, 1, 2)]),
]


@pytest.mark.parametrize("lattice,dim,S,steps", CHAINS)
def test_fused_chain_matches_oracle(abi, oracle, lattice, dim, S, steps):
    """scn_rules_chain_build (all layers in one kernel) against the oracle layer by layer."""
    rng = np.random.default_rng(S * 10 + dim)
    for dens, batch in (([0.02, 0.2, 0.6, 1.0, 0.0], 9), ([0.3], 300)):
        g = random_grids(rng, batch, dim, S, dens, triangular=(lattice == 1))
        dk, doff, dbg, _ = to_dev_grid(*g)
        regs, caps, n, bound = [], [], S, dk.numel()
        for size, stride, mn in steps:
            nOut = (n - size) // stride + 1
            regs.append(abi.regions(lattice, dim, n, nOut, size, stride, mn))
            T = 1 if mn == -1 else ((size + stride - 1) // stride) ** dim
            bound = min(bound * T, batch * nOut ** dim) + batch
            caps.append(bound)
            n = nOut
        max_rows = int(np.diff(g[2]).max() + 1)
        outs = abi.rules_chain_build(regs, dk, doff, dbg, max_rows, caps)
        assert outs is not None
        torch.cuda.synchronize()
        cur, n = g, S
        for (size, stride, mn), out in zip(steps, outs):
            nOut = (n - size) // stride + 1
            ref = oracle.grid_rules(lattice, dim, n, nOut, size, stride, mn, *cur)
            compare(out, out["result"].cpu().numpy(), ref)
            assert int(out["result"][3]) == int(np.diff(ref["out_off"]).max())
            cur = (ref["out_keys"], ref["out_rows"], ref["out_off"], ref["out_bg"])
            n = nOut


def test_resident_chain_matches_one_shot_build(abi, oracle):
    """scn_rules_chain_build_resident over a run of different batches (the device state of call n + 1 is prepared by the
    kernel of call n, the background rows are found by the kernel) against scn_rules_chain_build on the same grids: every
    output and every result record equal, call after call."""
    rng = np.random.default_rng(404)
    dim, S, batch = 2, 24, 37
    steps = [(3, 1, 1), (2, 2, 1), (2, 1, 2), (2, 2, 1)]
    regs, caps, n, bound = [], [], S, batch * (S * S + 1)
    for size, stride, mn in steps:
        nOut = (n - size) // stride + 1
        regs.append(abi.regions(0, dim, n, nOut, size, stride, mn))
        caps.append(batch * (nOut ** dim + 1))
        n = nOut
    chain = abi.ResidentChain(regs, batch, caps, torch.device("cuda"))
    for it, dens in enumerate(([0.3], [0.05, 0.9], [0.0, 1.0], [0.5], [0.2], [0.7, 0.1])):
        g = random_grids(rng, batch, dim, S, dens)
        dk, doff, dbg, _ = to_dev_grid(*g)
        max_rows = int(np.diff(g[2]).max() + 1)
        want = abi.rules_chain_build(regs, dk, doff, dbg, max_rows, caps)
        got = chain.build(dk, doff, None if it % 2 == 0 else dbg, max_rows)
        torch.cuda.synchronize()
        if it % 2 == 0:
            assert torch.equal(chain.bg, dbg)
        for a, b in zip(got, want):
            rows = int(b["result"][0])
            assert torch.equal(a["result"].cpu(), b["result"].cpu()), it
            assert torch.equal(a["out_off"], b["out_off"]) and torch.equal(a["out_bg"], b["out_bg"])
            assert torch.equal(a["out_keys"][:rows], b["out_keys"][:rows])
            assert torch.equal(a["rules"][: rows * a["sd"]], b["rules"][: rows * b["sd"]])


def test_fused_chain_declines_large_samples(abi):
    regs = [abi.regions(0, 3, 48, 46, 3, 1, 1)]
    z = torch.zeros(4, dtype=torch.int32, device="cuda")
    assert abi.rules_chain_build(regs, z, z[:2], z[:1], 6000, [200000]) is None


def test_fused_chain_row_hint(abi, oracle):
    """A hint sizes shared memory below the worst case: results are unchanged when it holds and
    SCN_DEV_ERR_CAPACITY is reported when a sample outgrows it."""
    rng = np.random.default_rng(77)
    dim, S, batch = 2, 20, 40
    g = random_grids(rng, batch, dim, S, [0.1, 0.5])
    dk, doff, dbg, _ = to_dev_grid(*g)
    regs = [abi.regions(0, dim, 20, 18, 3, 1, 1), abi.regions(0, dim, 18, 9, 2, 2, 1)]
    caps = [batch * (18 * 18 + 1), batch * (9 * 9 + 1)]
    max_rows = int(np.diff(g[2]).max() + 1)
    ref1 = oracle.grid_rules(0, dim, 20, 18, 3, 1, 1, *g)
    need = int(np.diff(ref1["out_off"]).max() + 1)
    good = abi.rules_chain_build(regs, dk, doff, dbg, max_rows, caps, rows_hint=need + 8)
    torch.cuda.synchronize()
    compare(good[0], good[0]["result"].cpu().numpy(), ref1)
    small = abi.rules_chain_build(regs, dk, doff, dbg, max_rows, caps, rows_hint=max_rows + 1)
    torch.cuda.synchronize()
    assert int(small[0]["result"][2]) & abi.DEV_ERR_CAPACITY


# Fractional max-pooling: (kind, dim, nOut, shrink), pool size 2; kinds 0/2 overlap, 1/3 do not.
FMP = [(k, d, n, s) for k in range(4) for d, n, s in [(1, 7, 1.414), (2, 5, 1.26), (2, 9, 1.7), (2, 24, 1.414), (3, 5, 1.26), (3, 12, 1.5)]]
FMP += [(1, 4, 3, 1.5), (3, 4, 3, 1.5), (0, 4, 3, 1.5)]


@pytest.mark.parametrize("kind,dim,nOut,shrink", FMP)
def test_fmp_rules(abi, oracle, kind, dim, nOut, shrink):
    """scn_fmp_rules_build against the oracle's restatement of the four FMP layers' preprocess, on the
    same tick tables (drawn by the oracle from a seeded copy of the reference's RNG)."""
    nIn = int(nOut * np.float32(shrink) + 0.5)
    nIn = nIn + 1 if nIn == nOut else nIn
    rng = np.random.default_rng(500 + 31 * kind + 7 * dim + nOut)
    for density in (0.0, 0.05, 0.4, 1.0):
        for with_bg in (True, False):
            g = random_grids(rng, 5, dim, nIn, density, with_bg=with_bg)
            ticks = oracle.fmp_ticks(kind, dim, nIn, nOut, 2, int(rng.integers(1, 2 ** 31)), 5)
            ref = oracle.fmp_rules(dim, nIn, nOut, 2, kind in (0, 2), ticks, *g)
            dk, doff, dbg, first = to_dev_grid(*g)
            assert first == 0
            cap = dk.numel() * 2 ** dim + len(g[3]) + 8
            out = abi.fmp_rules_build(dim, nIn, nOut, 2, kind in (0, 2), torch.from_numpy(ticks).cuda(), dk, doff, dbg, cap)
            torch.cuda.synchronize()
            compare(out, out["result"].cpu().numpy(), ref)
