"""The oracle's whole-network forward keeps every interface either from one pass over the batch or joined from
per-thread sample chunks; both must give the same numbering (row ids, rule cells, pooling choices, terminal
pooling rule width)."""
import numpy as np
import pytest


@pytest.mark.parametrize("cfg,batch", [(1, 7), (2, 5), (4, 5), (5, 3)])
def test_joined_chunks_equal_one_pass(scn, oracle, cfg, batch):
    from oracle import orc
    c = scn.synth.CONFIGS[cfg]
    net = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    scn.synth.build_network(net, cfg)
    for i, (W, B, pr) in scn.synth.init_weights(net.layers()).items():
        net.set_weights(i, W, B, pr)
    keys, off, feats = c["gen"](batch)
    p1, t1 = net.forward(keys, off, feats, keep=True, threads=1)
    one = [net.iface(i) for i in range(len(net.layers()) + 1)]
    p2, t2 = net.forward(keys, off, feats, keep=True, threads=3)
    joined = [net.iface(i) for i in range(len(net.layers()) + 1)]
    np.testing.assert_array_equal(p1, p2)
    np.testing.assert_array_equal(t1, t2)
    for i, (a, b) in enumerate(zip(one, joined)):
        for k in a:
            np.testing.assert_array_equal(a[k], b[k], err_msg="interface %d %s" % (i, k))


@pytest.mark.parametrize("name", ["POFMPSparseConvNet", "RDFMPSparseConvNet"])
def test_training_step_of_a_fractional_pooling_network_uses_the_forward_regions(scn, oracle, name):
    """orc_net_train_step draws the fractional max-pooling regions exactly as orc_net_forward does (same seed, same
    order): the step's probabilities are the forward's on the same weights, and repeated steps lower the loss."""
    from oracle import orc
    from netutil import build_named
    net = orc.OracleNet(oracle, 2, 3, 10, 1)
    build_named(net, name, 3, 32, orc.VLEAKYRELU, 0.0, 1.5)
    for i, (W, B, pr) in scn.synth.init_weights(net.layers(), 5).items():
        net.set_weights(i, W, B, None)
    net.seed_fmp(31)
    S = net.inputSpatialSize
    rng = np.random.default_rng(2)
    keys, feats, off = [], [], [0]
    for _ in range(4):
        kk = np.unique(rng.integers(0, S * S, 4 * S))
        keys.append(np.concatenate([[-1], kk]))
        feats.append(np.concatenate([np.zeros((1, 3)), rng.uniform(-1, 1, (len(kk), 3))]))
        off.append(off[-1] + len(kk) + 1)
    keys, off, feats = np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32)
    labels = np.arange(4, dtype=np.int32)
    fwd, _ = net.forward(keys, off, feats, accum64=True)
    probs, first = net.train_step(keys, off, feats, labels, 0.01, 0.9)
    np.testing.assert_array_equal(probs, fwd)
    last = first
    for _ in range(5):
        _, last = net.train_step(keys, off, feats, labels, 0.01, 0.9)
    assert np.isfinite(last["nll"]) and last["nll"] < first["nll"]
