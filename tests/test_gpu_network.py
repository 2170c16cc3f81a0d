"""GPU parity of whole networks: the C++ host classes (reference names) over the CUDA path
against the oracle, for the five benchmark configurations at reduced batch sizes.
Rulebooks, grids and pooling choices are compared bit-exactly, features and logits within
1e-4 relative (the fp32 / 3xTF32 tolerance), top-1 must agree."""
import numpy as np
import pytest
import torch

from netutil import make_pair, relerr

pytestmark = pytest.mark.gpu

RTOL = 1e-4
BATCH = {1: 6, 2: 3, 3: 2, 4: 3, 5: 1}


@pytest.fixture(scope="module")
def nets(scn, abi, oracle):
    cache = {}

    def get(cfg):
        if cfg not in cache:
            cache[cfg] = make_pair(scn, oracle, cfg)
        return cache[cfg]
    return get


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_builders_agree(scn, nets, cfg):
    gnet, onet = nets(cfg)
    gl, ol = gnet.layers(), onet.layers()
    assert len(gl) == len(ol)
    assert gnet.inputSpatialSize == onet.inputSpatialSize == scn.synth.CONFIGS[cfg]["grid"]
    for a, b in zip(gl, ol):
        assert a["type"] == b["type"]
        if a["type"] == 2:
            for k in ("nIn", "nOut", "act"):
                assert a[k] == b[k], (k, a, b)
            assert abs(a["dropout"] - b["dropout"]) < 1e-7
        else:
            for k in ("size", "stride", "fs", "inSpatial", "outSpatial"):
                assert a[k] == b[k], (k, a, b)
            if a["type"] in (0, 1):
                assert a["minActive"] == b["minActive"] and a["nIn"] == b["nIn"] and a["nOut"] == b["nOut"]


def test_deepcnet_builder_rounds_widths(scn, abi, oracle):
    """DeepCNet(2, 5, 100): widths 96/192/288/416/512/608, input field 127 (pool 3/2)."""
    from oracle import orc
    g = scn.net.Net.DeepCNet(2, 5, 100, abi.VLEAKYRELU, 3, 10, 0.5)
    o = orc.OracleNet.DeepCNet(oracle, 2, 5, 100, orc.VLEAKYRELU, 3, 10, 0.5)
    assert g.inputSpatialSize == o.inputSpatialSize == 127
    widths = [L["nOut"] for L in g.layers() if L["type"] == 2]
    assert widths == [96, 192, 288, 416, 512, 608, 10]
    for a, b in zip(g.layers(), o.layers()):
        assert a["type"] == b["type"] and abs(a["dropout"] - b["dropout"]) < 1e-7


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
@pytest.mark.parametrize("fusion", [False, True])
@pytest.mark.parametrize("precision", ["fp32", "auto", "3xtf32", "split", "3xbf16", "bf16"])
def test_forward_layer_by_layer(scn, abi, nets, cfg, precision, fusion):
    """Rulebooks and grids bit-exact; features of every interface and the probabilities within 1e-4 of
    the fp64-accumulating oracle for fp32 and the two split tensor-core precisions, within 2e-2 for the
    optional plain-bf16 precision; top-1 agrees (bf16: at least 99.9 % over the batch)."""
    gnet, onet = nets(cfg)
    gnet.set_precision(dict(fp32=abi.PREC_FP32, auto=abi.PREC_AUTO, split=abi.PREC_SPLIT, **{"3xtf32": abi.PREC_3XTF32, "3xbf16": abi.PREC_3XBF16},
                            bf16=abi.PREC_BF16)[precision])
    RTOL = 2e-2 if precision == "bf16" else 1e-4
    # fusion: convolution + learnt layer + non-overlapping pooling as one kernel (the default); the learnt layer's
    # own output is then never written, so only the run without fusion compares it
    gnet.set_pool_fusion(fusion)
    keys, off, feats = scn.synth.CONFIGS[cfg]["gen"](BATCH[cfg])
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
    # features and choices of the last pooled / learnt interfaces are still resident for the
    # interfaces that own a sub-interface; compare every one that is
    for i in range(1, len(layers) + 1):
        t = layers[i - 1]["type"]
        if t in (0, 1):
            continue
        try:
            g = gnet.iface(i)
        except abi.ScnError as e:
            assert fusion and t == 2 and "fused into the pooling layer" in str(e)
            continue
        o = onet.iface(i)
        assert relerr(g["features"], o["features"]) < RTOL, "features of interface %d" % i
    assert relerr(gprobs, oprobs) < RTOL
    if precision == "bf16":
        assert (gpred == opred).mean() >= 0.999 or (gpred != opred).sum() <= 1  # small batches: at most one near-tie may flip
    else:
        np.testing.assert_array_equal(gpred, opred)
    gnet.set_precision(abi.PREC_AUTO)
    gnet.set_pool_fusion(True)


@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_pooling_choices_fp32_equal_up_to_near_ties(scn, abi, nets, cfg):
    """Real-valued features: the fp32 kernels and the fp32 oracle add in different orders, so a choice may differ
    where two candidates lie within rounding of each other, and only there (the bit-exact comparison, on data that
    make the arithmetic exact, is test_gpu_benchmark_size.py::test_pooling_choices_bit_exact_on_integer_networks)."""
    gnet, onet = nets(cfg)
    gnet.set_precision(abi.PREC_FP32)
    keys, off, feats = scn.synth.CONFIGS[cfg]["gen"](BATCH[cfg])
    onet.forward(keys, off, feats, accum64=False, keep=True)
    gnet.forward_host(keys, off, feats)
    layers = gnet.layers()
    checked = 0
    for i in range(1, len(layers) + 1):
        if layers[i - 1]["type"] not in (3, 4):
            continue
        g, o = gnet.iface(i), onet.iface(i)
        gin, oin = gnet.iface(i - 1), onet.iface(i - 1)
        gc, oc = g["choices"], o["choices"]
        assert gc.shape == oc.shape
        same = gc == oc
        # where they differ the two candidates must be numerically tied within fp32 noise
        if not same.all():
            fin = oin["features"].ravel()
            d = np.abs(fin[gc[~same]] - fin[oc[~same]])
            assert d.max() <= 1e-5 * max(np.abs(fin).max(), 1.0)
        assert same.mean() > 0.999
        checked += 1
    assert checked > 0


def test_device_resident_forward_matches_host_path(scn, abi, nets):
    gnet, onet = nets(2)
    gnet.set_precision(abi.PREC_AUTO)
    keys, off, feats = scn.synth.CONFIGS[2]["gen"](5)
    probs, pred = gnet.forward_host(keys, off, feats)
    bg = np.array([off[b] for b in range(len(off) - 1)], np.int32)  # background row comes first
    dk, do, db, df = (torch.from_numpy(x).cuda() for x in (keys, off, bg, feats))
    dp, dt = gnet.forward_device(dk, do, db, df, max_sites=int(np.diff(off).max() - 1))
    torch.cuda.synchronize()
    np.testing.assert_array_equal(dp.cpu().numpy(), probs)
    np.testing.assert_array_equal(dt.cpu().numpy(), pred)


def test_process_dataset_with_batch_producer(scn, abi, nets):
    """SparseConvNetCUDA::processDataset over SitesPicture objects (producer threads, ragged
    last batch) gives the same probabilities as one direct forward."""
    gnet, onet = nets(1)
    gnet.set_precision(abi.PREC_AUTO)
    keys, off, feats = scn.synth.CONFIGS[1]["gen"](11)
    probs, pred = gnet.forward_host(keys, off, feats)
    labels = pred[:, 0].copy()
    labels[::4] = (labels[::4] + 1) % 10  # 3 of 11 wrong
    err, dprobs = gnet.process_dataset(keys, off, feats, labels, batch_size=4)
    np.testing.assert_allclose(dprobs, probs, rtol=1e-5, atol=1e-7)
    assert abs(err - 3.0 / 11.0) < 1e-6


def test_weight_file_round_trip(scn, abi, nets, tmp_path):
    """The .cnn file written by saveWeights is read by the oracle's loader and by loadWeights."""
    gnet, onet = nets(1)
    base = str(tmp_path / "w")
    gnet.save_weights(base, 3)
    c = scn.synth.CONFIGS[1]
    g2 = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    scn.synth.build_network(g2, 1)
    g2.load_weights(base, 3)
    from oracle import orc
    o2 = orc.OracleNet(onet.o, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    scn.synth.build_network(o2, 1)
    o2.load_weights(base + "_epoch-3.cnn")
    keys, off, feats = c["gen"](4)
    p1, _ = gnet.forward_host(keys, off, feats)
    p2, _ = g2.forward_host(keys, off, feats)
    p3, _ = o2.forward(keys, off, feats, accum64=True)
    np.testing.assert_array_equal(p1, p2)
    assert relerr(p1, p3) < RTOL
    with pytest.raises(abi.ScnError):
        g2.load_weights(str(tmp_path / "missing"), 0)


def test_multiply_add_count(scn, abi, nets):
    """multiplyAddCount = sum over learnt layers of rows x K x N, background rows included."""
    gnet, onet = nets(2)
    keys, off, feats = scn.synth.CONFIGS[2]["gen"](2)
    scn.net.take_multiply_adds()
    gnet.forward_host(keys, off, feats)
    got = scn.net.take_multiply_adds()
    layers = gnet.layers()
    want = 0
    for i, L in enumerate(layers):
        if L["type"] == 2:
            want += gnet.iface(i + 1, features=False)["nSpatialSites"] * L["nIn"] * L["nOut"]
    assert got == want
    assert abs(want / 2 - 81.9e6) < 0.2e6  # 81.9 M multiply-adds per sample with builder-rounded widths


def test_host_top_indices(scn, abi, oracle):
    rng = np.random.default_rng(1)
    for n, k in ((10, 1), (10, 3), (5, 5), (101, 5)):
        for _ in range(20):
            v = np.round(rng.standard_normal(n) * 2).astype(np.float32)
            np.testing.assert_array_equal(scn.net.host_top_indices(v, k), oracle.top_indices(v, k))


def test_alternating_batches_reuse_buffers(scn, abi, nets):
    """Every layer's buffers are reused from one forward to the next, and with dependent launches a kernel's
    set-up overlaps the end of the kernel in front of it: two different batches, alternated, must keep
    giving the bits of their first forwards (no stale feature, rule or partial-sum reads)."""
    gnet, _ = nets(2)
    gnet.set_precision(abi.PREC_AUTO)
    gnet.set_pool_fusion(True)
    gen = scn.synth.CONFIGS[2]["gen"]
    a, b = gen(24), gen(17, first=100)  # other inputs, other row counts
    first = [np.array(gnet.forward_host(*x)[0], copy=True) for x in (a, b)]
    assert not np.array_equal(first[0], first[1])
    for it in range(12):
        for x, want in zip((a, b), first):
            got = gnet.forward_host(*x)[0]
            assert np.array_equal(got, want), it


def test_begin_end_pipeline_equals_plain_calls(scn, abi, oracle):
    """forward_host in two halves: uploads run one batch ahead; results, order and the limit of two batches on their way."""
    c = scn.synth.CONFIGS[2]
    gnet, _ = make_pair(scn, oracle, 2)
    batches = [c["gen"](5 + (i % 3), first=10 * i) for i in range(6)]
    want = [gnet.forward_host(*b) for b in batches]
    with pytest.raises(scn.abi.ScnError):
        gnet.forward_host_end()  # nothing begun
    gnet.forward_host_begin(*batches[0])
    for i in range(len(batches)):
        if i + 1 < len(batches):
            gnet.forward_host_begin(*batches[i + 1])
            if i == 0:
                with pytest.raises(scn.abi.ScnError):
                    gnet.forward_host_begin(*batches[2])  # a third one
        probs, pred = gnet.forward_host_end()
        np.testing.assert_array_equal(probs, want[i][0])
        np.testing.assert_array_equal(pred, want[i][1])
    # the plain call still works behind the pipelined ones (and after a device-resident one)
    probs, pred = gnet.forward_host(*batches[1])
    np.testing.assert_array_equal(probs, want[1][0])
    assert abi.conv_tc_take_error() == 0
