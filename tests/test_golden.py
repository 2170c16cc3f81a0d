"""Golden vectors produced by the reference's own rule builder (tests/golden/make_golden.py):
checked against the oracle on CPU and against the CUDA path on the GPU, bit-exact."""
import os

import numpy as np
import pytest

G = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "rules_golden.npz"))
CASES = sorted({k.split("/")[0] for k in G.files if k.endswith("/params")})
FIELDS = ("rules", "out_keys", "out_rows", "out_off", "out_bg")
FMP_CASES = sorted({k.split("/")[0] for k in G.files if k.endswith("/fmp_params")})


def test_known_answer_8x8(oracle):
    """The hand-checkable example: conv3 on an 8x8 grid, then MP2 (vectorHash order)."""
    conv = G["known8x8_conv/rules"].reshape(-1, 9)
    assert conv.shape[0] == 28 and int(G["known8x8_conv/out_bg"][0]) == 27
    np.testing.assert_array_equal(conv[0], [0, 0, 0, 0, 0, 2, 0, 0, 3])
    np.testing.assert_array_equal(conv[5], [2, 0, 0, 3, 0, 0, 0, 0, 4])
    pool = G["known8x8_pool/rules"].reshape(-1, 4)
    np.testing.assert_array_equal(pool[:3], [[0, 1, 3, 4], [2, 27, 5, 9], [27, 27, 10, 27]])
    assert int(G["known8x8_pool/out_bg"][0]) == -1  # the pooled 3x3 grid is full
    a = oracle.grid_rules(0, 2, 8, 6, 3, 1, 1, G["known8x8_conv/in"], np.arange(1, 6), [0, 5], [0])
    b = oracle.grid_rules(0, 2, 6, 3, 2, 2, 1, a["out_keys"], a["out_rows"], a["out_off"], a["out_bg"])
    for f in FIELDS:
        np.testing.assert_array_equal(a[f], G["known8x8_conv/" + f])
        np.testing.assert_array_equal(b[f], G["known8x8_pool/" + f])


@pytest.mark.parametrize("name", CASES)
def test_oracle_matches_golden(oracle, name):
    lat, dim, nIn, nOut, size, stride, mn = (int(v) for v in G[name + "/params"])
    r = oracle.grid_rules(lat, dim, nIn, nOut, size, stride, mn, G[name + "/in_keys"], G[name + "/in_rows"],
                          G[name + "/in_off"], G[name + "/in_bg"])
    assert r["n_sites"] == int(G[name + "/n_sites"])
    for f in FIELDS:
        np.testing.assert_array_equal(r[f], G[name + "/" + f], err_msg=f)


@pytest.mark.gpu
@pytest.mark.parametrize("name", CASES)
def test_gpu_matches_golden(abi, name):
    import torch
    from test_gpu_rules import compare, run_gpu
    lat, dim, nIn, nOut, size, stride, mn = (int(v) for v in G[name + "/params"])
    g = (G[name + "/in_keys"], G[name + "/in_rows"], G[name + "/in_off"], G[name + "/in_bg"])
    out, res = run_gpu(abi, lat, dim, nIn, nOut, size, stride, mn, g)
    ref = {f: G[name + "/" + f] for f in FIELDS}
    ref["n_sites"] = int(G[name + "/n_sites"])
    compare(out, res, ref)
    torch.cuda.synchronize()


@pytest.mark.parametrize("name", FMP_CASES)
def test_oracle_fmp_matches_golden(oracle, name):
    """Tick tables (the reference's RNG, seeded) and FMP rulebooks as the reference build produced them."""
    kind, dim, nIn, nOut, ps, seed = (int(v) for v in G[name + "/fmp_params"])
    ticks = G[name + "/ticks"]
    np.testing.assert_array_equal(oracle.fmp_ticks(kind, dim, nIn, nOut, ps, seed, ticks.shape[0]), ticks)
    r = oracle.fmp_rules(dim, nIn, nOut, ps, kind in (0, 2), ticks, G[name + "/in_keys"], G[name + "/in_rows"], G[name + "/in_off"],
                         G[name + "/in_bg"])
    assert r["n_sites"] == int(G[name + "/n_sites"])
    for f in FIELDS:
        np.testing.assert_array_equal(r[f], G[name + "/" + f], err_msg=f)


@pytest.mark.gpu
@pytest.mark.parametrize("name", FMP_CASES)
def test_gpu_fmp_matches_golden(abi, name):
    import torch
    from test_gpu_rules import compare, to_dev_grid
    kind, dim, nIn, nOut, ps, seed = (int(v) for v in G[name + "/fmp_params"])
    g = (G[name + "/in_keys"], G[name + "/in_rows"], G[name + "/in_off"], G[name + "/in_bg"])
    dk, doff, dbg, first = to_dev_grid(*g)
    assert first == 0
    out = abi.fmp_rules_build(dim, nIn, nOut, ps, kind in (0, 2), torch.from_numpy(G[name + "/ticks"]).cuda(), dk, doff, dbg,
                              dk.numel() * ps ** dim + len(g[3]) + 8)
    torch.cuda.synchronize()
    ref = {f: G[name + "/" + f] for f in FIELDS}
    ref["n_sites"] = int(G[name + "/n_sites"])
    compare(out, out["result"].cpu().numpy(), ref)
