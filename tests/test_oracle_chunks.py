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
