"""GPU parity at the sizes the benchmark runs: whole networks at each configuration's own batch size with the
default settings (AUTO precision, pooling and classifier fusion, dependent launches, early first layer) through
both entry points, and single layers large enough that every CTA of the persistent tensor-core kernel walks
several work items (more than 148 row tiles), plain, with the pooling fused in and with two column tiles.

Integer-valued cases make the arithmetic exact (every product and partial sum is an integer that fp32, the
tf32 hi/lo split and the bf16 hi/lo split all represent exactly), so pooled values AND pooling choices must
equal the oracle's bit for bit whatever the summation order, ties included: the first maximum wins."""
import numpy as np
import pytest
import torch

from netutil import build_with, make_pair, relerr

pytestmark = pytest.mark.gpu

RTOL = 1e-4
BENCH_BATCH = {1: 32, 2: 256, 3: 64, 4: 64, 5: 64}


@pytest.fixture(scope="module")
def nets(scn, abi, oracle):
    cache = {}

    def get(cfg):
        if cfg not in cache:
            cache[cfg] = make_pair(scn, oracle, cfg)
        return cache[cfg]
    return get


def _device_inputs(keys, off, feats):
    bg = off[:-1].copy()  # the background row is each sample's first row
    return tuple(torch.from_numpy(np.ascontiguousarray(x)).cuda() for x in (keys, off, bg, feats)) + (int(np.diff(off).max() - 1),)


@pytest.mark.parametrize("entry", ["host", "device"])
@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_forward_at_benchmark_batch(scn, abi, nets, cfg, entry):
    """Every rulebook and grid bit-exact, pooled features and probabilities within 1e-4 of the fp64-accumulating
    oracle, top-1 equal, at the batch size the benchmark description gives the configuration."""
    gnet, onet = nets(cfg)
    gnet.set_precision(abi.PREC_AUTO)
    gnet.set_pool_fusion(True)
    keys, off, feats = scn.synth.CONFIGS[cfg]["gen"](BENCH_BATCH[cfg])
    oprobs, opred = onet.forward(keys, off, feats, accum64=True, keep=True, threads=16)
    if entry == "host":
        gprobs, gpred = gnet.forward_host(keys, off, feats)
    else:
        dk, do, db, df, ms = _device_inputs(keys, off, feats)
        dp, dt = gnet.forward_device(dk, do, db, df, ms)
        torch.cuda.synchronize()
        gprobs, gpred = dp.cpu().numpy(), dt.cpu().numpy()
    assert abi.conv_tc_take_error() == 0
    layers = gnet.layers()
    for i in range(len(layers) + 1):
        g, o = gnet.iface(i, features=False), onet.iface(i)
        assert g["nSpatialSites"] == o["nSpatialSites"], i
        np.testing.assert_array_equal(g["rules"], o["rules"], err_msg="rulebook of interface %d" % i)
        np.testing.assert_array_equal(g["row_keys"], o["row_keys"], err_msg="grid of interface %d" % i)
        if i and layers[i - 1]["type"] in (3, 4, 5):
            assert relerr(gnet.iface(i)["features"], o["features"]) < RTOL, "pooled features of interface %d" % i
    assert relerr(gprobs, oprobs) < RTOL
    np.testing.assert_array_equal(gpred, opred)


def test_top1_agreement_over_a_thousand_samples(scn, abi, oracle):
    """Top-1 agreement of at least 99.9 % over 1024 samples of the headline configuration whose predictions spread
    over the classes: the classifier's weights are drawn so that its logits are centred over the samples
    (random-normal weights alone send every sample to one class)."""
    gnet, onet = make_pair(scn, oracle, 2)
    layers = gnet.layers()
    gen = scn.synth.CONFIGS[2]["gen"]
    batches = [gen(256, first=5000 + 256 * j) for j in range(4)]
    top = len(layers) - 1
    hidden = []
    for keys, off, feats in batches:
        onet.forward(keys, off, feats, keep=True, threads=16)
        hidden.append(onet.iface(top)["features"].copy())
    hidden = np.concatenate(hidden)
    rng = np.random.default_rng(3)
    W2 = (rng.standard_normal((layers[top]["nIn"], layers[top]["nOut"])) * 4.0 / np.sqrt(layers[top]["nIn"])).astype(np.float32)
    B2 = (-(hidden.mean(0) @ W2)).astype(np.float32)
    scale = float(np.abs(hidden @ W2).max())  # size of the logits before the bias removes what all samples share
    onet.set_weights(top, W2, B2)
    gnet.set_weights(top, W2, B2)
    agree, total, seen = 0, 0, np.zeros(10, int)
    for keys, off, feats in batches:
        oprobs, opred = onet.forward(keys, off, feats, accum64=True, threads=16)
        gprobs, gpred = gnet.forward_host(keys, off, feats)
        # the bound is stated for the logits: compare them (up to the per-row constant that softmax removes) through log p,
        # relative to the logits' size before this test's bias centred them
        zo, zg = np.log(np.maximum(oprobs, 1e-30)), np.log(np.maximum(gprobs, 1e-30))
        zo, zg = zo - zo.mean(1, keepdims=True), zg - zg.mean(1, keepdims=True)
        assert float(np.abs(zg - zo).max()) / scale < RTOL
        agree += int((gpred == opred).sum())
        total += len(opred)
        seen += np.bincount(opred[:, 0], minlength=10)
    assert abi.conv_tc_take_error() == 0
    assert total == 1024 and agree / total >= 0.999
    assert (seen >= 20).sum() >= 6, seen  # predictions are spread: at least six classes take 2 % of the samples each


# ---------------------------------------------------------------------------------------------- single layers, many work items
BIG = [
    # rows_in, rows_out, fs, nIn, N, act, p           128-row tiles x column tiles
    (30000, 40000, 4, 96, 192, "VLEAKYRELU", 0.9),   # 313 items, A operand from tensor memory, two accumulators in turn
    (9000, 26000, 8, 96, 288, "VLEAKYRELU", 0.8),    # 204 row tiles x 2 column tiles of 144
    (20000, 21000, 1, 416, 416, "RELU", 1.0),        # plain learnt layer, 165 row tiles x 2 column tiles
    (40000, 60000, 9, 3, 96, "VLEAKYRELU", 0.9),     # first-layer form (row-per-lane gather), 469 items
]


@pytest.mark.parametrize("precision", ["3XTF32", "3XBF16", "SPLIT"])
@pytest.mark.parametrize("rows_in,rows_out,fs,nIn,N,act,p", BIG)
def test_conv_nin_many_items(abi, oracle, rows_in, rows_out, fs, nIn, N, act, p, precision):
    from oracle import orc
    prec = getattr(abi, "PREC_" + precision)
    rng = np.random.default_rng(rows_out + N)
    K = fs * nIn
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    if fs == 1:
        rows_out, rules, X = rows_in, None, feat
    else:
        rules = rng.integers(0, rows_in, size=(rows_out, fs)).astype(np.int32)
        rules[rng.random(rules.shape) < 0.05] = -1
        X = oracle.gather(feat, rules, nIn).reshape(rows_out, K)
    ref = oracle.nin_forward(X, W, B, None, p, getattr(orc, act), accum64=True)
    dW = torch.from_numpy(W).cuda()
    out = abi.conv_nin_forward(torch.from_numpy(feat).cuda(), None if rules is None else torch.from_numpy(rules).cuda().flatten(), fs, dW,
                               torch.from_numpy(B).cuda(), None, p, getattr(abi, act), prec, packed=abi.pack_weights(dW, prec))
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    assert relerr(out.cpu().numpy(), ref) < 5e-5


def _integer_layer(rng, rows_in, rows_mid, fs, nIn, N):
    K = fs * nIn
    feat = rng.integers(-8, 9, (rows_in, nIn)).astype(np.float32)
    W = rng.integers(-2, 3, (K, N)).astype(np.float32)
    B = rng.integers(-3, 4, N).astype(np.float32)
    rules = rng.integers(0, rows_in, size=(rows_mid, fs)).astype(np.int32)
    rules[rng.random(rules.shape) < 0.1] = -1
    return feat, W, B, rules


@pytest.mark.parametrize("rows_in,windows,fs,nIn,N,cells,split", [
    (30000, 10000, 4, 96, 192, 4, False),   # 313 work items: A from tensor memory, several items per CTA, pooling epilogue
    (9000, 6500, 8, 96, 288, 4, False),     # two column tiles
    (50000, 20000, 9, 3, 96, 4, False),     # first-layer form with two epilogue groups
    (20000, 5000, 27, 1, 32, 8, False),     # 3-D first layer, 2^3 windows
    (4000, 1024, 4, 416, 512, 4, True),     # K split over CTAs: pooling in the kernel that adds the partial sums
])
@pytest.mark.parametrize("precision", ["3XTF32", "SPLIT"])
def test_fused_pooling_choices_exact(abi, oracle, rows_in, windows, fs, nIn, N, cells, split, precision):
    """Convolution + learnt layer + max pooling as one kernel on integer data: pooled values and choices equal
    the oracle's bit for bit (MaxPoolingLayer.cu:17-33: negative rules skipped, first maximum wins, choice = row*C + j)."""
    from oracle import orc
    rng = np.random.default_rng(windows + N)
    rows_mid = windows * cells + 7
    feat, W, B, rules = _integer_layer(rng, rows_in, rows_mid, fs, nIn, N)
    pool = rng.permutation(rows_mid)[: windows * cells].astype(np.int32).reshape(windows, cells)
    pool[rng.random(pool.shape) < 0.1] = -1
    pool[11] = -1
    X = oracle.gather(feat, rules, nIn).reshape(rows_mid, fs * nIn)
    mid = oracle.nin_forward(X, W, B, None, 1.0, orc.VLEAKYRELU, accum64=False)
    assert np.array_equal(mid, oracle.nin_forward(X, W, B, None, 1.0, orc.VLEAKYRELU, accum64=True))  # the data are exact
    ref_v, ref_c = oracle.maxpool(mid, pool, cells)
    dW = torch.from_numpy(W).cuda()
    out, ch = abi.conv_nin_maxpool_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), fs, dW, torch.from_numpy(B).cuda(),
                                           torch.from_numpy(pool).cuda().flatten(), cells, None, 1.0, abi.VLEAKYRELU,
                                           abi.pack_weights(dW, getattr(abi, "PREC_" + precision)), rows_unpooled=rows_mid if split else 0, split_k=split,
                                           precision=getattr(abi, "PREC_" + precision))
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    out, ch = out.cpu().numpy(), ch.cpu().numpy()
    ok = ref_c >= 0  # windows without any input: the reference stores unset registers there, nothing to compare
    np.testing.assert_array_equal(ch[ok], ref_c[ok])
    np.testing.assert_array_equal(out[ok], ref_v[ok])
    assert (ch[~ok] == -1).all() and not out[~ok].any()
    assert (np.diff(np.sort(mid.reshape(-1))) == 0).any()  # the data do hold ties


@pytest.mark.parametrize("precision", ["FP32", "3XTF32", "3XBF16", "SPLIT"])
def test_learnt_layer_then_maxpool_exact_on_integers(abi, oracle, precision):
    """Separate kernels (learnt layer, then k_maxpool) on integer data: values and choices bit-exact in every precision."""
    from oracle import orc
    rng = np.random.default_rng(77)
    rows_in, windows, fs, nIn, N, cells = 6000, 5000, 4, 32, 96, 4
    rows_mid = windows * cells
    feat, W, B, rules = _integer_layer(rng, rows_in, rows_mid, fs, nIn, N)
    pool = rng.permutation(rows_mid).astype(np.int32).reshape(windows, cells)
    pool[rng.random(pool.shape) < 0.1] = -1
    pool[:, 0] = np.where(pool[:, 0] < 0, 3, pool[:, 0])
    X = oracle.gather(feat, rules, nIn).reshape(rows_mid, fs * nIn)
    mid = oracle.nin_forward(X, W, B, None, 1.0, orc.VLEAKYRELU, accum64=False)
    ref_v, ref_c = oracle.maxpool(mid, pool, cells)
    prec = getattr(abi, "PREC_" + precision)
    dW = torch.from_numpy(W).cuda()
    packed = None if precision == "FP32" else abi.pack_weights(dW, prec)
    dmid = abi.conv_nin_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), fs, dW, torch.from_numpy(B).cuda(), None, 1.0,
                                abi.VLEAKYRELU, prec, packed=packed)
    out, ch = abi.maxpool_forward(dmid, torch.from_numpy(pool).cuda().flatten(), cells)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    np.testing.assert_array_equal(dmid.cpu().numpy(), mid)
    np.testing.assert_array_equal(ch.cpu().numpy(), ref_c)
    np.testing.assert_array_equal(out.cpu().numpy(), ref_v)


# ---------------------------------------------------------------------------------------------- whole networks on integers
def _integer_weights(layers, seed):
    """Weights in {-1, 0, 1} with about six non-zeros per output column and biases in {-1, 0, 1}: with ReLU, no dropout and
    integer inputs every feature of every layer is an integer below 2^16, which both operand formats of the three-product
    split represent exactly (tf32: 11 + 11 bits, bf16: 8 + 8 bits)."""
    out = {}
    for i, L in enumerate(layers):
        if L["type"] != 2:
            continue
        rng = np.random.default_rng(seed + i)
        K, N = L["nIn"], L["nOut"]
        W = rng.integers(-1, 2, (K, N)).astype(np.float32) * (rng.random((K, N)) < min(1.0, 9.0 / K))
        out[i] = (W.astype(np.float32), rng.integers(-1, 2, N).astype(np.float32), None)
    return out


@pytest.mark.parametrize("precision", ["auto", "fp32"])
@pytest.mark.parametrize("cfg", [1, 2, 3, 4, 5])
def test_pooling_choices_bit_exact_on_integer_networks(scn, abi, oracle, cfg, precision):
    """poolingChoices (and pooled values) of every pooling layer equal the oracle's with array_equal, through the default
    fused kernels and through the fp32 kernels, at the benchmark's batch size (configuration 5: 16 samples)."""
    from oracle import orc
    c = scn.synth.CONFIGS[cfg]
    w = c["widths"]
    levels = []
    for i, nf in enumerate(w):
        pool = not (c["tail"] == "conv" and i == len(w) - 1)
        levels.append((nf, c.get("first_filter", 3) if i == 0 else 2, 1, 2 if pool else 1, 2 if pool else 1, orc.RELU, 0.0, 1))
    terminal = c.get("terminal") if c["tail"] == "terminal" else None
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(gnet, levels, terminal)
    layers = gnet.layers()
    for i, (W, B, pr) in _integer_weights(layers, 40 + cfg).items():
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    gnet.set_precision(abi.PREC_AUTO if precision == "auto" else abi.PREC_FP32)
    batch = 16 if cfg == 5 else BENCH_BATCH[cfg]
    keys, off, feats = c["gen"](batch)
    feats = np.round(feats * 3).astype(np.float32)
    onet.forward(keys, off, feats, accum64=False, keep=True, threads=16)
    gnet.forward_host(keys, off, feats)
    assert abi.conv_tc_take_error() == 0
    checked = 0
    for i, L in enumerate(layers):
        if L["type"] not in (3, 4):
            continue
        g, o = gnet.iface(i + 1), onet.iface(i + 1)
        assert np.abs(o["features"]).max() < 2 ** 16 and o["features"].any()  # exact in both operand formats of the split
        np.testing.assert_array_equal(g["choices"], o["choices"], err_msg="choices of pooling layer %d" % i)
        np.testing.assert_array_equal(g["features"], o["features"], err_msg="values of pooling layer %d" % i)
        checked += 1
    assert checked >= 3


def test_sample_larger_than_the_learnt_row_hint(scn, abi, nets):
    """The fused rule chain sizes its shared memory from the largest sample seen so far; a later batch with a much
    larger sample makes it report a capacity overflow, and the host rebuilds with the worst-case plan and reruns the
    layers that had started early.  Results must equal the oracle's as if nothing had happened."""
    gnet, onet = nets(1)
    gnet.set_precision(abi.PREC_AUTO)
    keys, off, feats = scn.synth.CONFIGS[1]["gen"](6)
    # the same samples cut down to their background row and first three sites
    sk, sf, so = [], [], [0]
    for b in range(6):
        sk.append(keys[off[b]:off[b] + 4]); sf.append(feats[off[b]:off[b] + 4]); so.append(so[-1] + 4)
    small = (np.concatenate(sk), np.array(so, np.int32), np.concatenate(sf))
    fresh, _ = make_pair(scn, onet.o, 1)  # a network that has seen no batch yet
    for data in (small, small, (keys, off, feats), small, (keys, off, feats)):
        gp, gt = fresh.forward_host(*data)
        op, ot = onet.forward(*data, accum64=True, keep=True)
        for i in range(len(fresh.layers()) + 1):
            np.testing.assert_array_equal(fresh.iface(i, features=False)["rules"], onet.iface(i)["rules"])
        assert relerr(gp, op) < RTOL
        np.testing.assert_array_equal(gt, ot)
