"""Fractional max-pooling networks (MaxPoolingLayer.cu:157-407; NetworkArchitectures.cpp:72-122) through
the C++ classes against the oracle: the same RNG seed gives the same region bounds, so rulebooks and
pooling choices are bit-exact and features agree within the fp32 tolerance."""
import numpy as np
import pytest

from netutil import relerr

pytestmark = pytest.mark.gpu

RTOL = 1e-4


def build_fmp(net, kind, dim, l, k, shrink, act, p=0.0):
    """The call sequence of {PO,RO,PD,RD}FMPSparseConvNet."""
    for i in range(l):
        net.addLeNetLayerFMP(kind, k * (i + 1), 2, 1, 2, shrink, act, p * i / (l + 1))
    net.addLeNetLayerMP(k * (l + 1), 2, 1, 1, 1, act, p * l / (l + 1))
    net.addLeNetLayerMP(k * (l + 2), 1, 1, 1, 1, act, p)
    net.addSoftmaxLayer()


def make_pair(scn, oracle, kind, dim, l, k, shrink, nIn=2, nClasses=7):
    from oracle import orc
    onet = orc.OracleNet(oracle, dim, nIn, nClasses, 1)
    gnet = scn.net.Net(dim, nIn, nClasses, 1, 0)
    build_fmp(onet, kind, dim, l, k, shrink, orc.VLEAKYRELU, 0.2)
    build_fmp(gnet, kind, dim, l, k, shrink, scn.abi.VLEAKYRELU, 0.2)
    for i, (W, B, pr) in scn.synth.init_weights(onet.layers()).items():
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    return gnet, onet


def random_batch(rng, batch, dim, S, nIn, density):
    keys, off, feats = [], [0], []
    for _ in range(batch):
        cells = np.flatnonzero(rng.random(S ** dim) < density)
        rng.shuffle(cells)
        keys.append(np.concatenate([[-1], cells]))  # the background row first
        f = rng.standard_normal((len(cells) + 1, nIn)).astype(np.float32)
        f[0] = 0
        feats.append(f)
        off.append(off[-1] + len(cells) + 1)
    return np.concatenate(keys).astype(np.int64), np.array(off, np.int32), np.concatenate(feats)


@pytest.mark.parametrize("kind", [0, 1, 2, 3])
@pytest.mark.parametrize("dim,l,k,shrink", [(2, 3, 32, 1.414), (2, 2, 32, 1.26), (3, 2, 32, 1.5)])
def test_fmp_network_layer_by_layer(scn, abi, oracle, kind, dim, l, k, shrink):
    gnet, onet = make_pair(scn, oracle, kind, dim, l, k, shrink)
    assert gnet.inputSpatialSize == onet.inputSpatialSize
    assert [L["type"] for L in gnet.layers()] == [L["type"] for L in onet.layers()]
    assert sum(L["type"] == 6 for L in gnet.layers()) == l
    rng = np.random.default_rng(kind + 10 * dim + l)
    for rep in range(2):  # a second batch re-seeded, then one continuing the RNG streams
        keys, off, feats = random_batch(rng, 5, dim, gnet.inputSpatialSize, 2, 0.15 if dim == 3 else 0.3)
        seed = int(rng.integers(1, 2 ** 31))
        gnet.seed_fmp(seed)
        onet.seed_fmp(seed)
        oprobs, opred = onet.forward(keys, off, feats, accum64=True, keep=True)
        gprobs, gpred = gnet.forward_host(keys, off, feats)
        layers = gnet.layers()
        for i in range(len(layers) + 1):
            g = gnet.iface(i, features=False)
            o = onet.iface(i)
            assert g["nSpatialSites"] == o["nSpatialSites"], i
            assert g["spatialSize"] == o["spatialSize"], i
            np.testing.assert_array_equal(g["rules"], o["rules"], err_msg="rules of interface %d" % i)
            np.testing.assert_array_equal(g["row_keys"], o["row_keys"], err_msg="grid of interface %d" % i)
            if i > 0 and layers[i - 1]["type"] not in (0, 1):
                assert relerr(gnet.iface(i)["features"], o["features"]) < RTOL, "features of interface %d" % i
        assert relerr(gprobs, oprobs) < RTOL
        np.testing.assert_array_equal(gpred, opred)


def test_fmp_threads_do_not_change_the_oracle(scn, abi, oracle):
    """The oracle draws every sample's region bounds before it splits the batch over threads."""
    gnet, onet = make_pair(scn, oracle, 0, 2, 2, 32, 1.414)
    rng = np.random.default_rng(5)
    keys, off, feats = random_batch(rng, 6, 2, onet.inputSpatialSize, 2, 0.3)
    onet.seed_fmp(77)
    a, _ = onet.forward(keys, off, feats, threads=1)
    b, _ = onet.forward(keys, off, feats, threads=3)
    np.testing.assert_array_equal(a, b)
