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


def build_with(net, levels, terminal=None):
    """levels: (nFeatures, filterSize, filterStride, poolSize, poolStride, activation, dropout, minActive) per
    addLeNetLayerMP call; then optional terminal pooling and the softmax layer."""
    for lv in levels:
        net.addLeNetLayerMP(*lv)
    if terminal:
        net.addTerminalPoolingLayer(terminal)
    net.addSoftmaxLayer()


def write_cnn(base, epoch, layers, weights):
    """A weight file as SparseConvNetCUDA::saveWeights lays it out (SparseConvNetCUDA.cu:425-442): per learnt layer W [K x N]
    then B [N] (NetworkInNetworkLayer.cu:308-323), for a PReLU layer the slopes behind them
    (NetworkInNetworkPReLULayer.cu:309-324); no momentum, no input normalising constants."""
    with open("%s_epoch-%d.cnn" % (base, epoch), "wb") as f:
        for i, L in enumerate(layers):
            if L["type"] != 2:
                continue
            W, B, pr = weights[i]
            f.write(np.ascontiguousarray(W, np.float32).tobytes())
            f.write(np.ascontiguousarray(B, np.float32).tobytes())
            if pr is not None:
                f.write(np.ascontiguousarray(pr, np.float32).tobytes())


def rules_safe_for_reference_kernels(onet):
    """The reference's gather kernel reads in front of its input for a rule of -1 and its pooling kernel stores unset
    registers for a row without any usable rule: true iff the last kept forward of the oracle has neither."""
    layers = onet.layers()
    for i, L in enumerate(layers):
        r = onet.iface(i + 1)["rules"]
        if L["type"] in (0, 1) and r.size and r.min() < 0:
            return False
        if L["type"] in (3, 4) and r.size and (r.reshape(-1, L["fs"]).max(axis=1) < 0).any():
            return False
    return True
