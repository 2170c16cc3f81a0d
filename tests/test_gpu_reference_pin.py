"""Pins the oracle to the reference's own network classes and CUDA kernels (oracle/_ref_gpu: the reference's
SparseConvNetCUDA, BatchProducer, layer classes, kernels and cuBLAS SGEMM compiled unchanged for this GPU).

For every layer of a network the oracle's layer function is fed the REFERENCE's input of that layer and its
result is compared with the reference's output: gather, max pooling values and choices bit-exact; learnt layers
(bias + SGEMM + dropout scaling + activation, PReLU, softmax) within 1e-5 of the largest output; terminal pooling
within 1e-6.  Rulebooks, grids, builder arithmetic (rounded widths, re-quantised dropout, input field size) and the
weight-file layout must be equal; probabilities, top-1, negative log-likelihood and mistakes of the whole network
must agree.  The product is then compared with the reference directly at the benchmark batch sizes."""
import numpy as np
import pytest

from netutil import build_with, relerr, rules_safe_for_reference_kernels, write_cnn

pytestmark = pytest.mark.gpu

GEMM_TOL = 1e-5


@pytest.fixture(scope="module")
def refgpu(abi):
    from oracle import orc
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built (it is compiled where the reference checkout is present)")
    return orc.ReferenceGPU


def _triple(scn, oracle, refgpu, tmp_path, dim, nIn, nClasses, lattice, build, seed=7, prelu=False, product=False):
    """The same network in the oracle, the reference and (optionally) the product, same weights through one .cnn file."""
    from oracle import orc
    onet = orc.OracleNet(oracle, dim, nIn, nClasses, 1, lattice=lattice)
    build(onet)
    ref = refgpu(dim, nIn, nClasses, 1, lattice)
    build(ref)
    layers = onet.layers()
    weights = scn.synth.init_weights(layers, seed)
    if prelu:
        for i, L in enumerate(layers):
            if L["type"] == 2 and L["act"] == orc.PRELU:
                W, B, _ = weights[i]
                weights[i] = (W, B, np.random.default_rng(100 + i).uniform(0.05, 0.5, L["nOut"]).astype(np.float32))
    for i, (W, B, pr) in weights.items():
        onet.set_weights(i, W, B, pr)
    base = str(tmp_path / "net")
    write_cnn(base, 1, layers, weights)
    ref.load_weights(base, 1)
    gnet = None
    if product:
        gnet = scn.net.Net(dim, nIn, nClasses, 1, lattice)
        build(gnet)
        gnet.load_weights(base, 1)
    return onet, ref, gnet, layers, weights


def _check_builders(onet, ref, layers):
    assert ref.inputSpatialSize == onet.inputSpatialSize
    rl = ref.layers()
    assert len(rl) == len(layers)
    for a, b in zip(layers, rl):
        assert (a["type"] == 2) == b["learnt"]
        if b["learnt"]:
            assert (a["nIn"], a["nOut"], a["act"]) == (b["nIn"], b["nOut"], b["act"]), (a, b)
            assert a["dropout"] == pytest.approx(b["dropout"], abs=1e-7)


def _check_layers(oracle, onet, ref, layers, weights, batch):
    """Oracle layer functions on the reference's inputs against the reference's outputs, rulebooks and grids."""
    from oracle import orc
    n = len(layers)
    R = [ref.iface(i) for i in range(n + 1)]
    worst = 0.0
    for i, L in enumerate(layers):
        o = onet.iface(i + 1)
        rin, rout = R[i], R[i + 1]
        assert rout["nSpatialSites"] == o["nSpatialSites"], i
        assert rout["spatialSize"] == o["spatialSize"], i
        np.testing.assert_array_equal(rout["row_keys"], o["row_keys"], err_msg="grid behind layer %d" % i)
        np.testing.assert_array_equal(rout["rules"], o["rules"], err_msg="rulebook of layer %d" % i)
        t = L["type"]
        if t in (0, 1):
            got = oracle.gather(rin["features"], rout["rules"], L["nIn"]).reshape(rout["features"].shape)
            np.testing.assert_array_equal(got, rout["features"], err_msg="gather of layer %d" % i)
        elif t == 2:
            W, B, pr = weights[i]
            for acc64 in (False, True):
                got = oracle.nin_forward(rin["features"], W, B, pr, p=1.0 - L["dropout"], act=L["act"], accum64=acc64)
                e = relerr(got, rout["features"])
                worst = max(worst, e)
                assert e < GEMM_TOL, "learnt layer %d (act %d, accum64 %s): %g" % (i, L["act"], acc64, e)
        elif t in (3, 4):
            v, ch = oracle.maxpool(rin["features"], rout["rules"], L["fs"])
            np.testing.assert_array_equal(v, rout["features"], err_msg="pooled values of layer %d" % i)
            np.testing.assert_array_equal(ch.ravel(), rout["choices"], err_msg="pooling choices of layer %d" % i)
        elif t == 5:
            S = rout["rules"].size // batch
            got = oracle.terminal_pool(rin["features"], rout["rules"], S)
            assert relerr(got, rout["features"]) < 1e-6, "terminal pooling"
    return worst


def _run(scn, oracle, refgpu, tmp_path, dim, nIn, nClasses, lattice, build, data, prelu=False, seed=7):
    onet, ref, _, layers, weights = _triple(scn, oracle, refgpu, tmp_path, dim, nIn, nClasses, lattice, build, seed, prelu)
    _check_builders(onet, ref, layers)
    keys, off, feats = data
    batch = len(off) - 1
    oprobs, opred = onet.forward(keys, off, feats, accum64=True, keep=True)
    assert rules_safe_for_reference_kernels(onet)
    labels = (np.arange(batch) % nClasses).astype(np.int32)
    rprobs, rpred, stats = ref.forward(keys, off, feats, labels=labels, batch_type=1)  # TESTBATCH
    worst = _check_layers(oracle, onet, ref, layers, weights, batch)
    assert relerr(oprobs, rprobs) < 1e-4
    np.testing.assert_array_equal(opred, rpred)
    nll = float(-np.log(np.maximum(oprobs[np.arange(batch), labels], 1e-15)).sum())
    assert stats["nll"] == pytest.approx(nll, rel=1e-4, abs=1e-4)
    assert stats["mistakes"] == int((opred[:, 0] != labels).sum())
    madds = sum(onet.iface(i + 1)["nSpatialSites"] * L["nIn"] * L["nOut"] for i, L in enumerate(layers) if L["type"] == 2)
    assert stats["multiply_adds"] == madds
    return worst


@pytest.mark.parametrize("cfg,batch", [(1, 8), (2, 4), (3, 2), (4, 3), (5, 1)])
def test_oracle_layers_match_reference_kernels(scn, oracle, refgpu, tmp_path, cfg, batch):
    c = scn.synth.CONFIGS[cfg]
    _run(scn, oracle, refgpu, tmp_path, c["dim"], c["nIn"], c["nClasses"], c["lattice"], lambda n: scn.synth.build_network(n, cfg),
         c["gen"](batch))


@pytest.mark.parametrize("act", ["NOSIGMOID", "RELU", "VLEAKYRELU", "LEAKYRELU", "TANH", "SIGMOID", "PRELU"])
def test_activations_match_reference_kernels(scn, oracle, refgpu, tmp_path, act):
    """Every activation the learnt layers offer (SigmoidLayer.cu:187-222, NetworkInNetworkPReLULayer.cu:8-23), with
    test-time dropout scaling, through a small 2-D network on pen-stroke inputs."""
    from oracle import orc
    a = getattr(orc, act)
    levels = [(32, 3, 1, 2, 2, a, 0.0, 1), (64, 2, 1, 2, 2, a, 0.2, 1), (96, 2, 1, 1, 1, a, 0.4, 1)]
    # 3 -> 2 -> 1 -> 1: input field 3 + ... is derived by addSoftmaxLayer; pictures are placed into a 48-grid only if it
    # matches, so derive the field from the oracle and draw sites inside it
    probe = orc.OracleNet(oracle, 2, 3, 10, 1)
    build_with(probe, levels)
    S = probe.inputSpatialSize
    rng = np.random.default_rng(5)
    keys, feats, off = [], [], [0]
    for s in range(6):
        k = np.unique(rng.integers(0, S * S, 3 * S))
        keys.append(np.concatenate([[-1], k]))
        feats.append(np.concatenate([np.zeros((1, 3)), rng.uniform(-1, 1, (len(k), 3))]))
        off.append(off[-1] + len(k) + 1)
    data = (np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32))
    _run(scn, oracle, refgpu, tmp_path, 2, 3, 10, 0, lambda n: build_with(n, levels), data, prelu=(act == "PRELU"))


def test_min_active_and_valid_builders_through_reference_layers(scn, oracle, refgpu, tmp_path):
    """minActiveInputs 2 (gridRulesOverlappingMin) and -1 (gridRulesValid, 3x3 in 2-D) through the reference's
    ConvolutionalLayer::preprocess."""
    from oracle import orc
    for levels in ([(32, 3, 1, 2, 2, orc.RELU, 0.0, 2), (32, 2, 1, 1, 1, orc.RELU, 0.0, 1)],
                   [(32, 3, 1, 2, 2, orc.RELU, 0.0, -1), (32, 2, 1, 1, 1, orc.RELU, 0.0, 1)]):
        probe = orc.OracleNet(oracle, 2, 2, 5, 1)
        build_with(probe, levels)
        S = probe.inputSpatialSize
        rng = np.random.default_rng(9)
        keys, feats, off = [], [], [0]
        for s in range(5):
            k = np.unique(rng.integers(0, S * S, S * S // 2))
            keys.append(np.concatenate([[-1], k]))
            feats.append(np.concatenate([np.zeros((1, 2)), rng.standard_normal((len(k), 2))]))
            off.append(off[-1] + len(k) + 1)
        data = (np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32))
        _run(scn, oracle, refgpu, tmp_path, 2, 2, 5, 0, lambda n: build_with(n, levels), data)


def test_product_weight_file_is_read_by_the_reference(scn, oracle, refgpu, tmp_path):
    """saveWeights of the product -> loadWeights of the reference -> the same numbers (PReLU slopes included)."""
    from oracle import orc
    levels = [(32, 3, 1, 2, 2, orc.PRELU, 0.0, 1), (64, 2, 1, 1, 1, orc.VLEAKYRELU, 0.0, 1)]
    gnet = scn.net.Net(2, 3, 10, 1, 0)
    build_with(gnet, levels)
    layers = gnet.layers()
    weights = scn.synth.init_weights(layers, 21)
    for i, (W, B, _) in weights.items():
        pr = np.random.default_rng(i).uniform(0.1, 0.4, len(B)).astype(np.float32) if layers[i]["act"] == orc.PRELU else None
        weights[i] = (W, B, pr)
        gnet.set_weights(i, W, B, pr)
    base = str(tmp_path / "w")
    gnet.save_weights(base, 2)
    ref = refgpu(2, 3, 10, 1, 0)
    build_with(ref, levels)
    ref.load_weights(base, 2)
    for i, (W, B, pr) in weights.items():
        rW, rB, rpr = ref.layer_weights(i)
        np.testing.assert_array_equal(rW, W)
        np.testing.assert_array_equal(rB, B)
        if pr is not None:
            np.testing.assert_array_equal(rpr, pr)
    ref.save_weights(str(tmp_path / "back"), 2)
    assert open(base + "_epoch-2.cnn", "rb").read() == open(str(tmp_path / "back") + "_epoch-2.cnn", "rb").read()


@pytest.mark.parametrize("cfg,batch", [(1, 32), (2, 256), (3, 64), (4, 64), (5, 16)])
def test_product_matches_reference_at_benchmark_batch(scn, abi, oracle, refgpu, tmp_path, cfg, batch):
    """The product with its default settings against the reference itself: rulebooks and grids equal, pooled features
    and probabilities within 1e-4, top-1 equal.  (Configuration 5 at 16 samples: the reference writes the gathered matrix
    of every convolution, which at 64 samples takes tens of GB and most of a minute.)"""
    c = scn.synth.CONFIGS[cfg]
    onet, ref, gnet, layers, weights = _triple(scn, oracle, refgpu, tmp_path, c["dim"], c["nIn"], c["nClasses"], c["lattice"],
                                               lambda n: scn.synth.build_network(n, cfg), product=True)
    keys, off, feats = c["gen"](batch)
    onet.forward(keys, off, feats, keep=True, threads=8)
    assert rules_safe_for_reference_kernels(onet)
    rprobs, rpred, _ = ref.forward(keys, off, feats)
    gprobs, gpred = gnet.forward_host(keys, off, feats)
    assert abi.conv_tc_take_error() == 0
    for i in range(len(layers) + 1):
        g, r = gnet.iface(i, features=False), ref.iface(i)
        assert g["nSpatialSites"] == r["nSpatialSites"], i
        np.testing.assert_array_equal(g["rules"], r["rules"], err_msg="rulebook of interface %d" % i)
        np.testing.assert_array_equal(g["row_keys"], r["row_keys"], err_msg="grid of interface %d" % i)
        if i and layers[i - 1]["type"] in (3, 4, 5):
            gf = gnet.iface(i)["features"]
            assert relerr(gf, r["features"]) < 1e-4, "pooled features of interface %d" % i
    assert relerr(gprobs, rprobs) < 1e-4
    np.testing.assert_array_equal(gpred, rpred)


@pytest.mark.parametrize("cfg,batch", [(1, 8), (2, 6), (4, 4)])
def test_rescale_batch_matches_the_reference(scn, abi, oracle, refgpu, tmp_path, cfg, batch):
    """RESCALEBATCH (SparseConvNetCUDA.cu:230-240, NetworkInNetworkLayer.cu:203-220): after one such batch every learnt
    layer's weights and biases equal the reference's; a forward afterwards gives the same probabilities."""
    c = scn.synth.CONFIGS[cfg]
    onet, ref, gnet, layers, weights = _triple(scn, oracle, refgpu, tmp_path, c["dim"], c["nIn"], c["nClasses"], c["lattice"],
                                               lambda n: scn.synth.build_network(n, cfg), product=True)
    keys, off, feats = c["gen"](batch)
    onet.forward(keys, off, feats, keep=True)
    assert rules_safe_for_reference_kernels(onet)
    ref.forward(keys, off, feats, batch_type=3)  # RESCALEBATCH
    gnet.rescale_batch(keys, off, feats)
    assert abi.conv_tc_take_error() == 0
    changed = False
    for i, L in enumerate(layers):
        if L["type"] != 2:
            continue
        rW, rB, _ = ref.layer_weights(i)
        gW, gB, _ = gnet.get_weights(i)
        assert relerr(gW, rW) < 1e-5, "weights of layer %d" % i
        assert relerr(gB, rB) < 1e-5, "biases of layer %d" % i
        changed = changed or relerr(gW, weights[i][0]) > 1e-3
    assert changed  # the pass did rescale something
    rprobs, rpred, _ = ref.forward(keys, off, feats)
    gprobs, gpred = gnet.forward_host(keys, off, feats)
    assert relerr(gprobs, rprobs) < 1e-4
    np.testing.assert_array_equal(gpred, rpred)
