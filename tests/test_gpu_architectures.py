"""The named architectures (NetworkArchitectures.h:4-69) constructed through their classes.

For each of DeepCNet, DeepC2, DeepCNiN, DeepC2C2, DeepC3C3Valid, DeepC3C3 and the four fractional max-pooling
networks: the layer list the class constructor leaves behind equals the oracle's (built from the same call sequence)
and the reference's (its own class, compiled test-only); one forward over seeded pictures gives equal rulebooks and
grids at every interface, probabilities within 1e-4 of the largest, the same top-1, and the negative log-likelihood
the reference reports for the batch."""
import numpy as np
import pytest

from netutil import NAMED_ARCHITECTURES, build_named, relerr, rules_safe_for_reference_kernels, write_cnn

pytestmark = pytest.mark.gpu

PROB_TOL = 1e-4
L_LEVELS, K_WIDTH, N_IN, N_CLASSES, BATCH = 3, 32, 3, 10, 6
FMP_SHRINK = 1.5


def _pictures(S, dim, nIn, batch, seed):
    rng = np.random.default_rng(seed)
    keys, feats, off = [], [], [0]
    for s in range(batch):
        k = np.unique(rng.integers(0, S ** dim, 4 * S))
        keys.append(np.concatenate([[-1], k]))
        feats.append(np.concatenate([np.zeros((1, nIn)), rng.uniform(-1, 1, (len(k), nIn))]))
        off.append(off[-1] + len(k) + 1)
    return np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32)


def _same_layers(a, b):
    """Per layer type the facts a builder decides: filter / pool geometry and field sizes, widths, activation, dropout."""
    assert len(a) == len(b)
    for i, (x, y) in enumerate(zip(a, b)):
        assert x["type"] == y["type"], (i, x, y)
        if x["type"] == 2:
            keys = ("nIn", "nOut", "act")
            assert x["dropout"] == pytest.approx(y["dropout"], abs=1e-7), (i, x, y)
        elif x["type"] in (0, 1):
            keys = ("size", "stride", "minActive", "nIn", "nOut", "fs", "inSpatial", "outSpatial")
        elif x["type"] == 5:
            keys = ("size",)
        else:
            keys = ("size", "stride", "fs", "inSpatial", "outSpatial")
        for key in keys:
            assert x[key] == y[key], (i, key, x, y)


@pytest.mark.parametrize("dropout", [0.0, 0.3])
@pytest.mark.parametrize("name", NAMED_ARCHITECTURES)
def test_named_architecture_matches_oracle_and_reference(scn, abi, oracle, tmp_path, name, dropout):
    from oracle import orc
    fmp = name.endswith("FMPSparseConvNet")
    shrink = FMP_SHRINK if fmp else 0.0
    act = orc.VLEAKYRELU
    gnet = scn.net.Net.named(name, 2, L_LEVELS, K_WIDTH, act, N_IN, N_CLASSES, p=dropout, fmpShrink=shrink)
    onet = orc.OracleNet(oracle, 2, N_IN, N_CLASSES, 1)
    build_named(onet, name, L_LEVELS, K_WIDTH, act, dropout, shrink)
    layers = onet.layers()
    _same_layers(gnet.layers(), layers)
    assert gnet.inputSpatialSize == onet.inputSpatialSize
    weights = scn.synth.init_weights(layers, 13)
    base = str(tmp_path / "w")
    write_cnn(base, 1, layers, weights)
    gnet.load_weights(base, 1)
    for i, (W, B, pr) in weights.items():
        onet.set_weights(i, W, B, pr)
    keys, off, feats = _pictures(onet.inputSpatialSize, 2, N_IN, BATCH, 17)
    labels = (np.arange(BATCH) % N_CLASSES).astype(np.int32)
    if fmp:
        gnet.seed_fmp(99)
        onet.seed_fmp(99)
    gprobs, gpred = gnet.forward_host(keys, off, feats)
    assert abi.conv_tc_take_error() == 0
    oprobs, opred = onet.forward(keys, off, feats, accum64=True, keep=True)
    n = len(layers)
    for i in range(n + 1):
        g, o = gnet.iface(i, features=False), onet.iface(i)
        assert g["nSpatialSites"] == o["nSpatialSites"], i
        np.testing.assert_array_equal(g["rules"], o["rules"], err_msg="rulebook of interface %d" % i)
        np.testing.assert_array_equal(g["row_keys"], o["row_keys"], err_msg="grid of interface %d" % i)
    assert relerr(gprobs, oprobs) < PROB_TOL
    np.testing.assert_array_equal(gpred, opred)
    nll = float(-np.log(np.maximum(gprobs[np.arange(BATCH), labels], 1e-15)).sum())
    onll = float(-np.log(np.maximum(oprobs[np.arange(BATCH), labels], 1e-15)).sum())
    assert nll == pytest.approx(onll, rel=1e-3, abs=1e-3)

    if not orc.ReferenceGPU.available():
        return
    ref = orc.ReferenceGPU(2, N_IN, N_CLASSES, 1, 0, named=(name, L_LEVELS, K_WIDTH, act, dropout, shrink))
    keys10 = ("type", "size", "stride", "minActive", "nIn", "nOut", "fs", "act", "inSpatial", "outSpatial")
    rl = [dict(zip(keys10, (int(v) for v in row))) for row in ref.describe()]
    for r, info in zip(rl, ref.layers()):
        r["dropout"] = info["dropout"]
    _same_layers(gnet.layers(), rl)
    assert ref.inputSpatialSize == gnet.inputSpatialSize
    if not rules_safe_for_reference_kernels(onet):
        pytest.skip("this batch holds a rule the reference's kernels read out of bounds for")
    ref.load_weights(base, 1)
    if fmp:
        ref.seed_fmp(99)
    rprobs, rpred, stats = ref.forward(keys, off, feats, labels=labels, batch_type=1)
    for i in range(n + 1):
        g, r = gnet.iface(i, features=False), ref.iface(i)
        assert g["nSpatialSites"] == r["nSpatialSites"], i
        np.testing.assert_array_equal(g["rules"], r["rules"], err_msg="reference rulebook of interface %d" % i)
        np.testing.assert_array_equal(g["row_keys"], r["row_keys"], err_msg="reference grid of interface %d" % i)
    assert relerr(gprobs, rprobs) < PROB_TOL
    np.testing.assert_array_equal(gpred, rpred)
    assert stats["nll"] == pytest.approx(nll, rel=1e-3, abs=1e-3)
    assert stats["mistakes"] == int((gpred[:, 0] != labels).sum())


def test_unknown_architecture_name_is_refused(scn):
    with pytest.raises(scn.abi.ScnError):
        scn.net.Net.named("DeepNothing", 2, 2, 32, 1, 3, 10)
