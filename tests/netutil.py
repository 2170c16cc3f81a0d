"""Build the same network in the product (C++ classes over CUDA) and in the oracle."""
import numpy as np


def make_pair(scn, oracle, cfg):
    from oracle import orc
    c = scn.synth.CONFIGS[cfg]
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    scn.synth.build_network(onet, cfg)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    scn.synth.build_network(gnet, cfg)
    weights = scn.synth.init_weights(onet.layers())
    for i, (W, B, pr) in weights.items():
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    return gnet, onet


def relerr(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))
