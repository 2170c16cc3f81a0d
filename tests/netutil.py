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
        if L["type"] in (3, 4, 6) and r.size and (r.reshape(-1, L["fs"]).max(axis=1) < 0).any():
            return False
    return True


NAMED_ARCHITECTURES = ("DeepCNet", "DeepC2", "DeepCNiN", "DeepC2C2", "DeepC3C3Valid", "DeepC3C3", "POFMPSparseConvNet",
                       "ROFMPSparseConvNet", "PDFMPSparseConvNet", "RDFMPSparseConvNet")


def build_named(net, name, l, k, fn, p=0.0, fmpShrink=0.0):
    """The builder calls the constructor of the named class makes (NetworkArchitectures.cpp:3-122), on any
    object that offers addLeNetLayerMP / addLeNetLayerFMP / addSoftmaxLayer.  Dropout arguments are float32
    products as in the C++ expressions."""
    f = np.float32
    ramp = lambda i, d: float(f(f(f(p) * f(i)) * f(1.0)) / f(d))
    mp = net.addLeNetLayerMP
    if name in ("DeepCNet", "DeepC2", "DeepCNiN"):
        for i in range(l + 1):
            last = i == l
            mp((i + 1) * k, 3 if (name == "DeepCNet" and i == 0) else 2, 1, 1 if last else 3, 1 if last else 2, fn, ramp(i, l), 1)
            if name == "DeepCNiN":
                mp((i + 1) * k, 1, 1, 1, 1, fn, ramp(i, l), 1)
    elif name in ("DeepC2C2", "DeepC3C3Valid", "DeepC3C3"):
        fs = 2 if name == "DeepC2C2" else 3
        ma = -1 if name == "DeepC3C3Valid" else 1
        for i in range(l):
            mp((i + 1) * k, fs, 1, 1, 1, fn, ramp(i, l), ma)
            mp((i + 1) * k, fs, 1, 3, 2, fn, ramp(i, l), ma)
        mp((l + 1) * k, fs, 1, 1, 1, fn, float(f(p)), 1)
        mp((l + 1) * k, 1, 1, 1, 1, fn, float(f(p)), 1)
    else:
        kind = {"PO": 0, "PD": 1, "RO": 2, "RD": 3}[name[:2]]
        for i in range(l):
            net.addLeNetLayerFMP(kind, k * (i + 1), 2, 1, 2, fmpShrink, fn, float(f(f(p) * f(i)) / f(l + 1)), 1)
        mp(k * (l + 1), 2, 1, 1, 1, fn, float(f(f(p) * f(l)) / f(l + 1)), 1)
        mp(k * (l + 2), 1, 1, 1, 1, fn, float(f(p)), 1)
    net.addSoftmaxLayer()
