"""GPU parity of the backward pass (the training step behind the forward path): every backward operation through
the C ABI against the oracle's restatement, one whole training step of the configurations' networks (without
dropout) against the oracle, the oracle's training step pinned to the reference's own TRAINBATCH branch
(its layer classes' backwards(), cuBLAS SGEMMs and SGD kernels compiled unchanged, oracle/_ref_gpu), and training
steps with dropout against that branch directly, on the feature subsets the reference drew."""
import numpy as np
import pytest
import torch

from netutil import build_with, relerr, rules_safe_for_reference_kernels, write_cnn

pytestmark = pytest.mark.gpu

TOL = 1e-4  # largest deviation relative to the largest value of a tensor (one operation, or a forward pass)
CHAIN_TOL = 1e-3  # the same for a gradient that has gone through a whole forward and backward pass (up to 13 chained contractions)
UPDATE_TOL = 5e-3  # weight updates of a whole step: sums over all rows of such gradients, the few near-tie decisions included


def dev(a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def grad_close(a, b, tol=CHAIN_TOL, outliers=1e-3):
    """Gradients of two runs of the same step: within tol of the largest value, except where a near-tie of the forward
    pass fell the other way in one of the runs (which input a pooling window chose, the side of zero of a leaky
    ReLU's input): there the gradient takes another route or another slope, a finite jump.  Such elements must be rare
    (at most `outliers` of all) and stay within the largest value itself."""
    a, b = np.asarray(a, np.float64).ravel(), np.asarray(b, np.float64).ravel()
    scale = max(float(np.abs(b).max()), 1e-30)
    diff = np.abs(a - b) / scale
    return bool((diff > tol).mean() <= outliers and diff.max() <= 1.0)


@pytest.mark.parametrize("act", ["NOSIGMOID", "RELU", "VLEAKYRELU", "LEAKYRELU", "TANH", "SIGMOID", "PRELU", "SOFTMAX"])
@pytest.mark.parametrize("rows,N", [(300, 96), (77, 10)])
def test_activation_backward(abi, oracle, act, rows, N):
    from oracle import orc
    rng = np.random.default_rng(N + len(act))
    a = getattr(orc, act)
    b = rng.standard_normal((rows, N)).astype(np.float32)
    if act in ("SIGMOID", "SOFTMAX"):
        b = (1 / (1 + np.exp(-b))).astype(np.float32)
    if act == "TANH":
        b = np.tanh(b).astype(np.float32)
    d = rng.standard_normal((rows, N)).astype(np.float32)
    pr = rng.uniform(0.1, 0.4, N).astype(np.float32) if act == "PRELU" else None
    want, wpr = oracle.activation_backward(b, d, a, pr)
    got, gpr = abi.activation_backward(dev(b), dev(d), a, None if pr is None else dev(pr))
    assert relerr(got.cpu().numpy(), want) < 1e-6
    if act == "PRELU":
        assert relerr(gpr.cpu().numpy(), wpr) < 1e-5


@pytest.mark.parametrize("rows_in,rows,fs,nIn,N", [
    (300, 257, 9, 3, 32), (500, 1000, 4, 96, 192), (64, 64, 1, 160, 10), (200, 513, 27, 1, 32), (90, 77, 4, 50, 101),
    (3000, 5000, 8, 32, 64), (256, 256, 1, 608, 10), (2000, 3000, 1, 70, 33),
])
def test_conv_nin_backward_weights(abi, oracle, rows_in, rows, fs, nIn, N):
    """dW = X^T d, dB = column sums, the gathered matrix read through the rulebook inside the kernel."""
    rng = np.random.default_rng(rows + N)
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    d = rng.standard_normal((rows if fs > 1 else rows_in, N)).astype(np.float32)
    if fs > 1:
        rules = rng.integers(0, rows_in, size=(rows, fs)).astype(np.int32)
        rules[rng.random(rules.shape) < 0.1] = -1
        X = oracle.gather(feat, rules, nIn).reshape(rows, fs * nIn)
        drules = dev(rules).flatten()
    else:
        X, drules = feat, None
    W = np.zeros((X.shape[1], N), np.float32)
    wdW, wdB, _ = oracle.nin_backward(X, d, W, want_dx=False)
    gdW, gdB = abi.conv_nin_backward_weights(dev(feat), drules, fs, dev(d))
    assert relerr(gdW.cpu().numpy(), wdW) < TOL
    assert relerr(gdB.cpu().numpy(), wdB) < TOL


@pytest.mark.parametrize("rows_in,rows,fs,nIn,N", [
    (300, 257, 9, 3, 32), (500, 1000, 4, 96, 192), (200, 513, 27, 1, 32), (90, 177, 4, 50, 100), (3000, 5000, 8, 32, 64),
    (2000, 3000, 1, 70, 36), (256, 256, 1, 2048, 608), (20000, 40000, 4, 96, 192), (9000, 70001, 9, 3, 96),
])
def test_conv_nin_backward_weights_on_tensor_cores(abi, oracle, rows_in, rows, fs, nIn, N):
    """The same gradient as the forward kernel's product with the roles turned (gathered input transposed, gradient packed
    as the weight operand, contraction over the rows split over the CTAs): within 1e-4 of the largest entry."""
    rng = np.random.default_rng(rows + N)
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    d = rng.standard_normal((rows if fs > 1 else rows_in, N)).astype(np.float32)
    if fs > 1:
        rules = rng.integers(0, rows_in, size=(rows, fs)).astype(np.int32)
        rules[rng.random(rules.shape) < 0.1] = -1
        X = oracle.gather(feat, rules, nIn).reshape(rows, fs * nIn)
        drules = dev(rules).flatten()
    else:
        X, drules = feat, None
    wdW = (X.astype(np.float64).T @ d.astype(np.float64)).astype(np.float32)
    wdB = d.astype(np.float64).sum(axis=0).astype(np.float32)
    gdW, gdB = abi.conv_nin_backward_weights_tc(dev(feat), drules, fs, dev(d))
    assert abi.conv_tc_take_error() == 0
    assert relerr(gdW.cpu().numpy(), wdW) < TOL
    assert relerr(gdB.cpu().numpy(), wdB) < TOL
    sdW, sdB = abi.conv_nin_backward_weights(dev(feat), drules, fs, dev(d))  # the CUDA-core form agrees
    assert relerr(gdW.cpu().numpy(), sdW.cpu().numpy()) < TOL


def test_tensor_core_weight_gradient_refuses_small_shapes(abi):
    feat, d = torch.zeros((64, 32), device="cuda"), torch.zeros((64, 10), device="cuda")
    with pytest.raises(abi.ScnError):
        abi.conv_nin_backward_weights_tc(feat, None, 1, d)


@pytest.mark.parametrize("precision", ["FP32", "3XTF32"])
@pytest.mark.parametrize("rows,K,N", [(1000, 384, 192), (300, 96, 32), (256, 608, 10), (5000, 1152, 416)])
def test_input_gradient_is_the_forward_kernel_on_transposed_weights(abi, oracle, rows, K, N, precision):
    """dX = d W^T through scn_transpose_weights + scn_conv_nin_forward_ws (tensor cores where the shape allows)."""
    rng = np.random.default_rng(K + N)
    d = rng.standard_normal((rows, N)).astype(np.float32)
    W = (rng.standard_normal((K, N)) / np.sqrt(K)).astype(np.float32)
    _, _, want = oracle.nin_backward(np.zeros((rows, K), np.float32), d, W)
    Wt = abi.transpose_weights(dev(W))
    np.testing.assert_array_equal(Wt.cpu().numpy(), W.T)
    prec = getattr(abi, "PREC_" + precision)
    packed = None
    if precision != "FP32":
        if abi.lib().scn_conv_packed_weight_bytes(N, K, prec) == 0:
            pytest.skip("no tensor-core layout for this shape")
        packed = abi.pack_weights(Wt, prec)
    got = abi.conv_nin_forward(dev(d), None, 1, Wt, torch.zeros(K, device="cuda"), None, 1.0, abi.NOSIGMOID, prec, packed=packed)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    assert relerr(got.cpu().numpy(), want) < TOL


def test_gather_backward(abi, oracle):
    rng = np.random.default_rng(5)
    rows_in, rows, fs, nIn = 400, 700, 9, 24
    rules = rng.integers(0, rows_in, size=(rows, fs)).astype(np.int32)
    rules[rng.random(rules.shape) < 0.2] = -1
    dconv = rng.standard_normal((rows * fs, nIn)).astype(np.float32)
    want = oracle.gather_backward(dconv, rules, nIn, rows_in)
    got = abi.gather_backward(dev(dconv), dev(rules).flatten(), nIn, rows_in)
    assert relerr(got.cpu().numpy(), want) < 1e-5


def test_maxpool_backward(abi, oracle):
    """Overlapping windows: several pooled values may choose the same input, their gradients add up."""
    rng = np.random.default_rng(6)
    n_in, n = 5000, 3000
    choices = rng.integers(0, n_in // 4, n).astype(np.int32)  # many duplicates
    choices[rng.random(n) < 0.05] = -1
    dout = rng.standard_normal(n).astype(np.float32)
    want = oracle.maxpool_backward(dout, choices, n_in)
    got = abi.maxpool_backward(dev(dout), dev(choices), n_in)
    assert relerr(got.cpu().numpy(), want) < 1e-5


def test_terminal_pool_backward(abi, oracle):
    rng = np.random.default_rng(7)
    C, S, batch, rows_in = 96, 9, 17, 200
    rules = np.full((batch, S), -1, np.int32)
    perm = rng.permutation(rows_in)
    at = 0
    for b in range(batch):
        n = int(rng.integers(1, S + 1))
        rules[b, :n] = perm[at:at + n]
        at += n
    dout = rng.standard_normal((batch, C)).astype(np.float32)
    want = oracle.terminal_pool_backward(dout, rules, S, rows_in)
    got = abi.terminal_pool_backward(dev(dout), dev(rules).flatten(), S, rows_in)
    np.testing.assert_allclose(got.cpu().numpy(), want, rtol=1e-6, atol=1e-7)


def test_softmax_nll_backward_and_sgd_update(abi, oracle):
    rng = np.random.default_rng(8)
    p = rng.random((64, 10)).astype(np.float32)
    p /= p.sum(1, keepdims=True)
    labels = rng.integers(0, 10, 64).astype(np.int32)
    got = abi.softmax_nll_backward(dev(p), dev(labels)).cpu().numpy()
    want = p.copy()
    want[np.arange(64), labels] -= 1
    np.testing.assert_array_equal(got, want)
    w, m, d = (rng.standard_normal(5000).astype(np.float32) for _ in range(3))
    ww, wm = oracle.sgd_update(w, m, d, 0.003, 0.99)
    gw, gm = dev(w), dev(m)
    abi.sgd_update(gw, gm, dev(d), 0.003, 0.99)
    np.testing.assert_allclose(gw.cpu().numpy(), ww, rtol=1e-6, atol=1e-7)
    np.testing.assert_allclose(gm.cpu().numpy(), wm, rtol=1e-6, atol=1e-7)
    ww, wm = oracle.sgd_update(w, m, d, 0.5, 0.9, keep_positive=True)  # the PReLU slopes' update: held at 0.001 or above
    gw, gm = dev(w), dev(m)
    abi.sgd_update(gw, gm, dev(d), 0.5, 0.9, keep_positive=True)
    np.testing.assert_allclose(gw.cpu().numpy(), ww, rtol=1e-6, atol=1e-6)
    assert gw.min().item() >= 0.001 and (gw == 0.001).any().item()


def test_mask_columns_and_masked_update(abi, oracle):
    """The two operations training-time dropout adds: zeroing the dropped features' columns, and the SGD update that
    leaves every entry of a dropped input feature (row mask, periodic over a convolution's copies) or output feature
    (column mask) bit-identical while the others move exactly as scn_sgd_update moves them."""
    rng = np.random.default_rng(9)
    x = rng.standard_normal((301, 40)).astype(np.float32)
    cm = (rng.uniform(size=40) < 0.6).astype(np.float32)
    gx = dev(x)
    abi.mask_columns(gx, dev(cm))
    np.testing.assert_array_equal(gx.cpu().numpy(), x * cm)
    nIn, copies, N = 12, 4, 40
    rm = (rng.uniform(size=nIn) < 0.5).astype(np.float32)
    w, m, d = (rng.standard_normal((nIn * copies, N)).astype(np.float32) for _ in range(3))
    for row_mask, col_mask in ((rm, cm), (None, cm), (rm, None)):
        ww, wm = oracle.sgd_update(w.ravel(), m.ravel(), d.ravel(), 0.05, 0.9)
        keep = np.ones((nIn * copies, N), bool)
        if row_mask is not None:
            keep &= np.tile(row_mask, copies)[:, None] != 0
        if col_mask is not None:
            keep &= col_mask[None, :] != 0
        gw, gm = dev(w), dev(m)
        abi.sgd_update_masked(gw, gm, dev(d), None if row_mask is None else dev(row_mask), nIn, None if col_mask is None else dev(col_mask), 0.05, 0.9)
        plain_w, plain_m = dev(w), dev(m)
        abi.sgd_update(plain_w, plain_m, dev(d), 0.05, 0.9)
        np.testing.assert_array_equal(gw.cpu().numpy(), np.where(keep, plain_w.cpu().numpy(), w))
        np.testing.assert_array_equal(gm.cpu().numpy(), np.where(keep, plain_m.cpu().numpy(), m))
        np.testing.assert_allclose(gw.cpu().numpy()[keep], ww.reshape(w.shape)[keep], rtol=1e-6, atol=1e-6)


# ---------------------------------------------------------------------------------------------- whole training steps
def _levels(scn, cfg, act):
    c = scn.synth.CONFIGS[cfg]
    w = c["widths"]
    out = []
    for i, nf in enumerate(w):
        pool = not (c["tail"] == "conv" and i == len(w) - 1)
        out.append((nf, c.get("first_filter", 3) if i == 0 else 2, 1, 2 if pool else 1, 2 if pool else 1, act, 0.0, 1))
    return out, (c.get("terminal") if c["tail"] == "terminal" else None)


def _compare_step(gnet, onet, layers, old):
    """dfeatures of every interface a gradient reaches and every learnt layer's update, product against oracle."""
    checked = 0
    for i in range(len(layers) + 1):
        o = onet.dfeatures(i)
        if i and layers[i - 1]["type"] in (0, 1):
            continue  # the gathered matrix's gradient is never materialised by the fused kernels
        g = gnet.dfeatures(i)
        if o.size == 0:
            continue
        assert g.size == o.size, "gradient of interface %d" % i
        assert grad_close(g, o), "gradient of interface %d: %g" % (i, relerr(g, o))
        checked += 1
    for i, L in enumerate(layers):
        if L["type"] != 2:
            continue
        gW, gB, gpr = gnet.get_weights(i)
        oW, oB, opr = onet.get_weights(i)
        W0, B0, pr0 = old[i]
        assert relerr(gW - W0, oW - W0) < UPDATE_TOL, "weight update of layer %d" % i
        assert relerr(gB - B0, oB - B0) < UPDATE_TOL, "bias update of layer %d" % i
        if opr is not None:
            assert relerr(gpr - pr0, opr - pr0) < UPDATE_TOL, "slope update of layer %d" % i  # a sum over the rows on the negative side only
    return checked


@pytest.mark.parametrize("cfg,batch,act", [(1, 16, "VLEAKYRELU"), (2, 32, "VLEAKYRELU"), (3, 6, "RELU"), (4, 6, "PRELU"), (5, 2, "VLEAKYRELU"), (1, 8, "TANH")])
def test_training_step_matches_oracle(scn, abi, oracle, cfg, batch, act):
    """Two consecutive training steps (the second runs on updated weights and non-zero momentum) of each configuration's
    network built without dropout: probabilities, negative log-likelihood, the gradient at every interface and every
    weight update within 1e-4 of the fp64-accumulating oracle."""
    from oracle import orc
    c = scn.synth.CONFIGS[cfg]
    levels, terminal = _levels(scn, cfg, getattr(orc, act))
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(gnet, levels, terminal)
    layers = gnet.layers()
    weights = scn.synth.init_weights(layers, 11)
    for i, (W, B, _) in weights.items():
        pr = np.random.default_rng(i).uniform(0.1, 0.4, len(B)).astype(np.float32) if layers[i]["act"] == orc.PRELU else None
        weights[i] = (W, B, pr)
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    for step in range(2):
        keys, off, feats = c["gen"](batch, first=100 * step)
        labels = ((np.arange(batch) * 7 + step) % c["nClasses"]).astype(np.int32)
        old = {i: onet.get_weights(i) for i in weights}
        oprobs, ostats = onet.train_step(keys, off, feats, labels, 0.01, 0.9)
        gprobs, gstats = gnet.train_batch(keys, off, feats, labels, 0.01, 0.9)
        assert abi.conv_tc_take_error() == 0
        assert relerr(gprobs, oprobs) < TOL
        assert gstats["nll"] == pytest.approx(ostats["nll"], rel=1e-4)
        assert gstats["mistakes"] == ostats["mistakes"]
        assert _compare_step(gnet, onet, layers, old) >= 3
    # the updated network still forwards like the oracle's
    keys, off, feats = c["gen"](batch, first=500)
    op, ot = onet.forward(keys, off, feats, accum64=True)
    gp, gt = gnet.forward_host(keys, off, feats)
    assert relerr(gp, op) < TOL


def test_training_with_dropout_draws_the_reference_number_of_features(scn, abi):
    """Without forced subsets every learnt layer of a network built with dropout keeps floor(nOut (1 - dropout)) randomly
    drawn output features per TRAINBATCH (NetworkInNetworkLayer.cu:152-154), another draw each batch, zero elsewhere; the
    weights of dropped features do not move; and test-time forwards keep every feature."""
    gnet = scn.net.Net(2, 3, 10, 1, 0)
    scn.synth.build_network(gnet, 2)  # dropout ramp 0 .. 0.5
    layers = gnet.layers()
    keys, off, feats = scn.synth.CONFIGS[2]["gen"](4)
    labels = np.arange(4, dtype=np.int32)
    learnt = [i for i, L in enumerate(layers) if L["type"] == 2]
    draws = []
    for step in range(2):
        old = {i: gnet.get_weights(i) for i in learnt}
        gnet.train_batch(keys, off, feats, labels, 0.01, 0.9)
        assert abi.conv_tc_take_error() == 0
        draws.append({})
        for i in learnt:
            L = layers[i]
            present = gnet.iface_present(i + 1)
            want = int(np.float32(L["nOut"]) * (np.float32(1.0) - np.float32(L["dropout"])))
            assert len(present) == want and (np.diff(present) > 0).all() and present.max() < L["nOut"]
            draws[-1][i] = present
            dropped = np.setdiff1d(np.arange(L["nOut"]), present)
            f = gnet.iface(i + 1)["features"]
            assert not f[:, dropped].any()
            W, B, _ = gnet.get_weights(i)
            assert (W[:, dropped] == old[i][0][:, dropped]).all() and (B[dropped] == old[i][1][dropped]).all()
            assert (W[:, present] != old[i][0][:, present]).any()
    assert any(len(draws[0][i]) != len(np.intersect1d(draws[0][i], draws[1][i])) for i in learnt), "the same subsets twice"
    gnet.forward_host(keys, off, feats)
    for i in learnt:
        assert len(gnet.iface_present(i + 1)) == layers[i]["nOut"]


def test_prelu_slopes_of_dropped_features_do_not_move(scn, abi):
    """A PReLU layer with dropout: a training batch updates the slopes of the features it keeps and leaves the others
    bit-identical.  (No reference result exists for this case: NetworkInNetworkPReLULayer.cu:199 tests
    `size() < size()`, never true, and so runs its full-width slope update on the narrow gradient vector.)"""
    from oracle import orc
    gnet = scn.net.Net(2, 3, 10, 1, 0)
    build_with(gnet, [(32, 3, 1, 2, 2, orc.PRELU, 0.0, 1), (64, 2, 1, 2, 2, orc.PRELU, 0.5, 1), (96, 2, 1, 2, 2, orc.PRELU, 0.5, 1)], None)
    layers = gnet.layers()
    S = gnet.inputSpatialSize
    rng = np.random.default_rng(3)
    pts = [np.unique(rng.integers(0, S * S, 40)) for _ in range(4)]
    keys = np.concatenate(pts).astype(np.int32)
    off = np.concatenate([[0], np.cumsum([len(p) for p in pts])]).astype(np.int32)
    feats = rng.standard_normal((len(keys), 3)).astype(np.float32)
    old = {i: gnet.get_weights(i) for i, L in enumerate(layers) if L["type"] == 2}
    gnet.train_batch(keys, off, feats, np.arange(4, dtype=np.int32), 0.05, 0.9)
    assert abi.conv_tc_take_error() == 0
    seen = 0
    for i, (W0, B0, pr0) in old.items():
        if pr0 is None or layers[i]["dropout"] == 0:
            continue
        present = gnet.iface_present(i + 1)
        dropped = np.setdiff1d(np.arange(layers[i]["nOut"]), present)
        pr = gnet.get_weights(i)[2]
        assert len(dropped) and (pr[dropped] == pr0[dropped]).all()
        assert (pr[present] != pr0[present]).any()
        seen += 1
    assert seen == 2


def _reference_dropout_steps(abi, ref, gnet, onet, layers, weights, gen, batch, nClasses, min_dropped=2):
    """Two TRAINBATCHes of the reference (weights already loaded) against the product with the subsets the reference drew;
    `gen(step)` gives the samples of a step, `onet` (same layers) only checks that the rulebooks are safe for the reference's
    kernels.  See test_training_steps_with_dropout_match_reference for what is compared."""
    nL = len(layers)
    for i, (W, B, pr) in weights.items():  # the oracle runs the same steps: its restatement of dropout is pinned here too
        onet.set_weights(i, W, B, pr)
    ref.seed_dropout(1234)  # (the reference seeds these generators from the clock)
    lr, mom = 0.01, 0.9
    dropped_somewhere = 0
    for step in range(2):
        keys, off, feats = gen(step)
        labels = ((np.arange(batch) * 3 + step) % nClasses).astype(np.int32)
        onet.forward(keys, off, feats, keep=True)
        assert rules_safe_for_reference_kernels(onet)
        before = {i: gnet.get_weights(i) for i in weights}
        rbefore = {i: ref.layer_weights(i) for i in weights}
        rprobs, _, rstats = ref.forward(keys, off, feats, labels=labels, batch_type=0, learning_rate=lr, momentum=mom)
        order = ref.sample_numbers(batch)
        R = [ref.iface(i) for i in range(nL + 1)]
        # cols[i]: the features interface i keeps (of its full width), as the reference's featuresPresent lists them
        cols = [R[i]["present"] if R[i]["featuresPresent"] else np.arange(R[i]["nFeatures"]) for i in range(nL + 1)]
        for i, L in enumerate(layers):
            if L["type"] == 2:
                gnet.set_dropout_features(i, cols[i + 1] if len(cols[i + 1]) < L["nOut"] else [])
                onet.set_dropout_features(i, cols[i + 1])
                dropped_somewhere += len(cols[i + 1]) < L["nOut"]
        k2 = np.concatenate([keys[off[s]:off[s + 1]] for s in order])
        f2 = np.concatenate([feats[off[s]:off[s + 1]] for s in order])
        o2 = np.concatenate([[0], np.cumsum([off[s + 1] - off[s] for s in order])]).astype(np.int32)
        l2 = labels[order]
        gprobs, gstats = gnet.train_batch(k2, o2, f2, l2, lr, mom)
        assert abi.conv_tc_take_error() == 0
        assert relerr(gprobs, rprobs) < TOL
        assert gstats["nll"] == pytest.approx(rstats["nll"], rel=1e-4)
        assert gstats["mistakes"] == rstats["mistakes"]
        obefore = {i: onet.get_weights(i) for i in weights}
        oprobs, ostats = onet.train_step(k2, o2, f2, l2, lr, mom)
        assert relerr(oprobs, rprobs) < TOL and ostats["nll"] == pytest.approx(rstats["nll"], rel=1e-4) and ostats["mistakes"] == rstats["mistakes"]
        for i in weights:
            oW, oB, _ = onet.get_weights(i)
            rW, rB, _ = ref.layer_weights(i)
            assert relerr(oW - obefore[i][0], rW - rbefore[i][0]) < 4 * UPDATE_TOL, "oracle's weight update of layer %d" % i
            assert relerr(oB - obefore[i][1], rB - rbefore[i][1]) < 4 * UPDATE_TOL, "oracle's bias update of layer %d" % i
        checked = 0
        tie_above = nL + 2  # the highest interface at which a near-tie of the forward pass fell the other way (see grad_close)
        for i in range(nL, -1, -1):
            if i and layers[i - 1]["type"] in (0, 1):
                continue  # the gathered matrix is never materialised by the fused kernels
            G = gnet.iface(i)
            assert (gnet.iface_present(i) == cols[i]).all() if (i and layers[i - 1]["type"] == 2) else True
            rows, nF = G["nSpatialSites"], G["nFeatures"]
            gone = np.setdiff1d(np.arange(nF), cols[i])
            rf = R[i]["features"]
            if rf.size:
                assert rf.shape == (rows, len(cols[i])), "reference features of interface %d" % i
                assert relerr(G["features"][:, cols[i]], rf) < TOL, "features of interface %d" % i
                assert not G["features"][:, gone].any(), "dropped features of interface %d" % i
            rd = R[i]["dfeatures"]
            if rd.size:
                gd = gnet.dfeatures(i).reshape(rows, nF)
                # (one near-tie that falls the other way in a learnt layer above spreads over a whole row here, and these
                # batches have few hundred rows: hence 1 % of the elements, not 0.1 %)
                assert grad_close(gd[:, cols[i]], rd, outliers=1e-2), "gradient of interface %d: %g" % (i, relerr(gd[:, cols[i]], rd))
                assert not gd[:, gone].any(), "gradient of the dropped features of interface %d" % i
                if tie_above > nL and not grad_close(gd[:, cols[i]], rd, outliers=0.0):
                    tie_above = i
                checked += 1
        assert checked >= 3
        for i in weights:
            L = layers[i]
            W0, B0, _ = before[i]
            rW0, rB0, _ = rbefore[i]
            rW, rB, _ = ref.layer_weights(i)
            gW, gB, _ = gnet.get_weights(i)
            rows_in = cols[i]  # the convolution in front lists present + copy * nIn for every copy (ConvolutionalLayer.cu:117-127)
            keep = np.zeros(W0.shape, bool)
            keep[np.ix_(rows_in, cols[i + 1])] = True
            assert (gW[~keep] == W0[~keep]).all() and (rW[~keep] == rW0[~keep]).all(), "weights of dropped features of layer %d" % i
            # (a near-tie at or above this layer's output puts one row's gradient on another slope or route: with the
            # few hundred rows of these batches that is up to a percent or two of a weight gradient)
            tol = UPDATE_TOL if i + 1 > tie_above else 4 * UPDATE_TOL
            assert relerr((gW - W0)[keep], (rW - rW0)[keep]) < tol, "weight update of layer %d" % i
            gone = np.setdiff1d(np.arange(L["nOut"]), cols[i + 1])
            assert (gB[gone] == B0[gone]).all() and (rB[gone] == rB0[gone]).all()
            assert relerr((gB - B0)[cols[i + 1]], (rB - rB0)[cols[i + 1]]) < tol, "bias update of layer %d" % i
    assert dropped_somewhere >= min_dropped


@pytest.mark.parametrize("cfg,batch,act", [(1, 8, "VLEAKYRELU"), (2, 4, "RELU"), (3, 2, "LEAKYRELU"), (5, 1, "TANH")])
def test_training_steps_with_dropout_match_reference(scn, abi, oracle, tmp_path, cfg, batch, act):
    """Two TRAINBATCHes of the reference's own processBatch on a network with a dropout ramp, against the product's
    training step on the same samples (in the order the reference shuffled them into) with the feature subsets the
    reference drew.  The reference narrows every matrix to the kept features; the product keeps full widths with zeros.
    Compared: probabilities, NLL, the kept columns of the features and of the gradient at every materialised interface
    (the dropped ones must be zero), and the weights after each step: the entries that touch a dropped input or output
    feature must be bit-identical to before, the others within the update tolerance."""
    from oracle import orc
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built")
    c = scn.synth.CONFIGS[cfg]
    levels, terminal = _levels(scn, cfg, getattr(orc, act))
    levels = [lv[:6] + (0.1 * i,) + lv[7:] for i, lv in enumerate(levels)]  # dropout 0, 0.1, 0.2, ...
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    ref = orc.ReferenceGPU(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(ref, levels, terminal)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(gnet, levels, terminal)
    layers = gnet.layers()
    nL = len(layers)
    weights = scn.synth.init_weights(layers, 17)
    for i, (W, B, _) in weights.items():
        weights[i] = (W, B, None)
        gnet.set_weights(i, W, B, None)
    base = str(tmp_path / "t")
    write_cnn(base, 0, layers, weights)
    ref.load_weights(base, 0)
    _reference_dropout_steps(abi, ref, gnet, onet, layers, weights, lambda step: c["gen"](batch, first=50 * step), batch, c["nClasses"])


@pytest.mark.parametrize("cfg,batch,act", [(1, 8, "VLEAKYRELU"), (2, 4, "RELU"), (3, 2, "LEAKYRELU"), (4, 3, "PRELU"), (5, 1, "TANH"), (1, 6, "SIGMOID")])
def test_oracle_backward_operations_match_reference(scn, abi, oracle, tmp_path, cfg, batch, act):
    """The oracle's backward pass pinned to the reference, operation by operation: one TRAINBATCH through the reference's own
    processBatch (forward, SoftmaxClassifier, every layer's backwards with its cuBLAS SGEMMs and SGD kernels), then every
    oracle backward operation is fed the REFERENCE's tensors of the interface above (features, pooling choices, rules, the
    gradient it left there) and must reproduce the gradient the reference left one interface below, and the weight update of
    every learnt layer.  No error accumulates from layer to layer and the forward pass's decisions (pooling choices, signs)
    are the reference's own."""
    from oracle import orc
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built")
    c = scn.synth.CONFIGS[cfg]
    levels, terminal = _levels(scn, cfg, getattr(orc, act))
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    ref = orc.ReferenceGPU(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(ref, levels, terminal)
    layers = onet.layers()
    nL = len(layers)
    weights = scn.synth.init_weights(layers, 13)
    for i, (W, B, _) in weights.items():
        pr = np.random.default_rng(i).uniform(0.1, 0.4, len(B)).astype(np.float32) if layers[i]["act"] == orc.PRELU else None
        weights[i] = (W, B, pr)
        onet.set_weights(i, W, B, pr)
    base = str(tmp_path / "t")
    write_cnn(base, 0, layers, weights)
    ref.load_weights(base, 0)
    keys, off, feats = c["gen"](batch)
    labels = ((np.arange(batch) * 3) % c["nClasses"]).astype(np.int32)
    onet.forward(keys, off, feats, keep=True)
    assert rules_safe_for_reference_kernels(onet)
    lr, mom = 0.5, 0.9  # a large rate: the update is read back as w_new - w_old and must stand clear of the weights' own rounding
    rprobs, _, rstats = ref.forward(keys, off, feats, labels=labels, batch_type=0, learning_rate=lr, momentum=mom)
    order = ref.sample_numbers(batch)
    l2 = labels[order]
    R = [ref.iface(i) for i in range(nL + 1)]
    backprop = [False] + [False] * nL
    for i, L in enumerate(layers):
        backprop[i + 1] = True if L["type"] == 2 else backprop[i]
    # raw[i]: the gradient the layer above interface i hands down, computed by the oracle from the reference's tensors
    raw = {nL: rprobs.copy()}
    raw[nL][np.arange(batch), l2] -= 1  # SoftmaxClassifier.cu:7-14
    step = lr * (1 - mom) * (1 + mom)   # first step, zero momentum: w_new - w_old = -lr (1 - momentum)(1 + momentum) dW
    checked = 0
    for i in range(nL, 0, -1):
        L = layers[i - 1]
        got = R[i]["dfeatures"]
        want = raw.get(i)
        if want is None:
            continue
        if L["type"] == 2:  # the learnt layer under interface i rescales it in place by the activation's derivative
            want, dpr = oracle.activation_backward(R[i]["features"], want.reshape(R[i]["features"].shape), L["act"], weights[i - 1][2])
        assert got.size == want.size, "gradient of interface %d" % i
        assert relerr(want, got.reshape(want.shape)) < TOL, "gradient the reference left at interface %d" % i
        checked += 1
        d = got.reshape(want.shape)
        rows_in = R[i - 1]["nSpatialSites"]
        if L["type"] == 2:
            W0, B0, pr0 = weights[i - 1]
            dW, dB, dX = oracle.nin_backward(R[i - 1]["features"], d, W0, want_dx=backprop[i - 1])
            rW, rB, rpr = ref.layer_weights(i - 1)
            # the update is read back as w_new - w_old: where gradients vanish (saturating activations) it is no larger than a
            # few units in the last place of the weights themselves, which then bounds what can be seen of it
            seen = lambda w0, dw: TOL + 2 * 6e-8 * float(np.abs(w0).max()) / max(float(np.abs(dw).max()), 1e-30)
            assert relerr(-step * dW, rW - W0) < seen(W0, rW - W0), "weight update of layer %d" % (i - 1)
            assert relerr(-step * dB, rB - B0) < seen(B0, rB - B0), "bias update of layer %d" % (i - 1)
            if pr0 is not None:
                assert relerr(np.maximum(pr0 - step * dpr, 0.001) - pr0, rpr - pr0) < TOL, "slope update of layer %d" % (i - 1)
            if backprop[i - 1]:
                raw[i - 1] = dX
        elif not backprop[i - 1]:
            continue
        elif L["type"] in (0, 1):
            raw[i - 1] = oracle.gather_backward(d.reshape(-1, L["nIn"]), R[i]["rules"], L["nIn"], rows_in)
        elif L["type"] in (3, 4):
            raw[i - 1] = oracle.maxpool_backward(d, R[i]["choices"], rows_in * L["nIn"])
        elif L["type"] == 5:
            raw[i - 1] = oracle.terminal_pool_backward(d.reshape(batch, -1), R[i]["rules"], R[i]["rules"].size // batch, rows_in)
    assert checked >= 5


@pytest.mark.parametrize("cfg,batch,act", [(1, 8, "VLEAKYRELU"), (2, 4, "RELU"), (4, 3, "PRELU")])
def test_training_step_matches_reference(scn, abi, oracle, tmp_path, cfg, batch, act):
    """One whole TRAINBATCH of the reference (its own processBatch) against orc_net_train_step and against the product's
    training step on the same samples, in the order the reference's BatchProducer shuffled them into: gradients at every
    interface, updated weights, NLL, mistakes."""
    from oracle import orc
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built")
    c = scn.synth.CONFIGS[cfg]
    levels, terminal = _levels(scn, cfg, getattr(orc, act))
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    ref = orc.ReferenceGPU(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(ref, levels, terminal)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(gnet, levels, terminal)
    layers = onet.layers()
    weights = scn.synth.init_weights(layers, 13)
    for i, (W, B, _) in weights.items():
        pr = np.random.default_rng(i).uniform(0.1, 0.4, len(B)).astype(np.float32) if layers[i]["act"] == orc.PRELU else None
        weights[i] = (W, B, pr)
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    base = str(tmp_path / "t")
    write_cnn(base, 0, layers, weights)
    ref.load_weights(base, 0)
    keys, off, feats = c["gen"](batch)
    labels = ((np.arange(batch) * 3) % c["nClasses"]).astype(np.int32)
    onet.forward(keys, off, feats, keep=True)
    assert rules_safe_for_reference_kernels(onet)
    lr, mom = 0.01, 0.9
    rprobs, _, rstats = ref.forward(keys, off, feats, labels=labels, batch_type=0, learning_rate=lr, momentum=mom)
    order = ref.sample_numbers(batch)
    # the same samples in the reference's order
    k2 = np.concatenate([keys[off[s]:off[s + 1]] for s in order])
    f2 = np.concatenate([feats[off[s]:off[s + 1]] for s in order])
    o2 = np.concatenate([[0], np.cumsum([off[s + 1] - off[s] for s in order])]).astype(np.int32)
    l2 = labels[order]
    oprobs, ostats = onet.train_step(k2, o2, f2, l2, lr, mom)
    gprobs, gstats = gnet.train_batch(k2, o2, f2, l2, lr, mom)
    assert relerr(oprobs, rprobs) < TOL and relerr(gprobs, rprobs) < TOL
    assert rstats["nll"] == pytest.approx(ostats["nll"], rel=1e-4)
    assert rstats["mistakes"] == ostats["mistakes"] == gstats["mistakes"]
    checked = 0
    for i in range(len(layers) + 1):
        r = ref.iface(i)["dfeatures"].ravel()
        o = onet.dfeatures(i)
        if o.size == 0:
            continue
        assert r.size == o.size, "gradient of interface %d" % i
        assert grad_close(o, r), "oracle gradient of interface %d: %g" % (i, relerr(o, r))
        if not (i and layers[i - 1]["type"] in (0, 1)):
            assert grad_close(gnet.dfeatures(i), r), "product gradient of interface %d" % i
        checked += 1
    assert checked >= 3
    for i, (W0, B0, pr0) in weights.items():
        rW, rB, rpr = ref.layer_weights(i)
        oW, oB, opr = onet.get_weights(i)
        gW, gB, gpr = gnet.get_weights(i)
        assert relerr(oW - W0, rW - W0) < UPDATE_TOL and relerr(gW - W0, rW - W0) < UPDATE_TOL, "weight update of layer %d" % i
        assert relerr(oB - B0, rB - B0) < UPDATE_TOL and relerr(gB - B0, rB - B0) < UPDATE_TOL, "bias update of layer %d" % i
        if pr0 is not None:
            assert relerr(opr - pr0, rpr - pr0) < UPDATE_TOL and relerr(gpr - pr0, rpr - pr0) < UPDATE_TOL, "slope update of layer %d" % i


@pytest.mark.parametrize("name", ["DeepCNet", "DeepC2", "DeepCNiN", "DeepC2C2", "DeepC3C3Valid", "DeepC3C3"])
def test_named_architectures_train_with_dropout_like_the_reference(scn, abi, oracle, tmp_path, name):
    """The same comparison for the named classes (NetworkArchitectures.cpp:3-70) built with their dropout ramp: learnt
    layers that follow learnt layers directly (DeepCNiN), two convolutions per level (DeepC2C2, DeepC3C3) and the
    valid-convolution builder (DeepC3C3Valid) put the dropped features in front of layers without a gather, behind two
    of them, and in front of a convolution that drops sites."""
    from oracle import orc
    from netutil import build_named
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built")
    l, k, nIn, nClasses, batch, p = 3, 32, 3, 10, 6, 0.4
    act = orc.VLEAKYRELU
    gnet = scn.net.Net.named(name, 2, l, k, act, nIn, nClasses, p=p)
    onet = orc.OracleNet(oracle, 2, nIn, nClasses, 1)
    build_named(onet, name, l, k, act, p)
    ref = orc.ReferenceGPU(2, nIn, nClasses, 1, 0, named=(name, l, k, act, p, 0.0))
    layers = gnet.layers()
    weights = scn.synth.init_weights(layers, 19)
    for i, (W, B, _) in weights.items():
        weights[i] = (W, B, None)
        gnet.set_weights(i, W, B, None)
    base = str(tmp_path / "t")
    write_cnn(base, 0, layers, weights)
    ref.load_weights(base, 0)
    S = gnet.inputSpatialSize

    def gen(step):
        rng = np.random.default_rng(100 + step)
        keys, feats, off = [], [], [0]
        for _ in range(batch):
            kk = np.unique(rng.integers(0, S * S, 4 * S))
            keys.append(np.concatenate([[-1], kk]))
            feats.append(np.concatenate([np.zeros((1, nIn)), rng.uniform(-1, 1, (len(kk), nIn))]))
            off.append(off[-1] + len(kk) + 1)
        return np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32)

    _reference_dropout_steps(abi, ref, gnet, onet, layers, weights, gen, batch, nClasses, min_dropped=1)


@pytest.mark.parametrize("name", ["POFMPSparseConvNet", "ROFMPSparseConvNet", "PDFMPSparseConvNet", "RDFMPSparseConvNet"])
def test_fractional_max_pooling_networks_train_like_the_oracle(scn, abi, oracle, name):
    """Two training steps of the four fractional max-pooling classes (NetworkArchitectures.cpp:72-122, no dropout; both sides
    draw their pooling regions from the same seeded generators): the backward pass routes gradients through the pooling
    choices of overlapping and disjoint, pseudorandom and random regions (MaxPoolingLayer.cu:187-199 and its siblings)."""
    from oracle import orc
    from netutil import build_named
    l, k, nIn, nClasses, batch, shrink = 3, 32, 3, 10, 5, 1.5
    act = orc.VLEAKYRELU
    gnet = scn.net.Net.named(name, 2, l, k, act, nIn, nClasses, p=0.0, fmpShrink=shrink)
    onet = orc.OracleNet(oracle, 2, nIn, nClasses, 1)
    build_named(onet, name, l, k, act, 0.0, shrink)
    layers = gnet.layers()
    weights = scn.synth.init_weights(layers, 23)
    for i, (W, B, _) in weights.items():
        weights[i] = (W, B, None)
        onet.set_weights(i, W, B, None)
        gnet.set_weights(i, W, B, None)
    onet.seed_fmp(77)
    S = gnet.inputSpatialSize
    for step in range(2):
        gnet.seed_fmp(77)  # (the oracle seeds its generators anew for every batch)
        rng = np.random.default_rng(300 + step)
        keys, feats, off = [], [], [0]
        for _ in range(batch):
            kk = np.unique(rng.integers(0, S * S, 4 * S))
            keys.append(np.concatenate([[-1], kk]))
            feats.append(np.concatenate([np.zeros((1, nIn)), rng.uniform(-1, 1, (len(kk), nIn))]))
            off.append(off[-1] + len(kk) + 1)
        keys, off, feats = np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32)
        labels = ((np.arange(batch) * 7 + step) % nClasses).astype(np.int32)
        old = {i: onet.get_weights(i) for i in weights}
        oprobs, ostats = onet.train_step(keys, off, feats, labels, 0.01, 0.9)
        gprobs, gstats = gnet.train_batch(keys, off, feats, labels, 0.01, 0.9)
        assert abi.conv_tc_take_error() == 0
        assert relerr(gprobs, oprobs) < TOL
        assert gstats["nll"] == pytest.approx(ostats["nll"], rel=1e-4)
        for i in range(len(layers) + 1):
            np.testing.assert_array_equal(gnet.iface(i, features=False)["rules"], onet.iface(i)["rules"], err_msg="rulebook of interface %d" % i)
        assert _compare_step(gnet, onet, layers, old) >= 3


def test_training_step_at_benchmark_batch_on_both_kernel_families(scn, abi):
    """Config 2 at its benchmark batch of 256 (dropout 0), one training step twice: with the default kernels (tensor cores:
    forward, input gradients and weight gradients through the fused kernel) and with every learnt layer set to plain fp32
    (CUDA-core kernels, the ones the small cases above compare with the oracle, which needs minutes at this size).  Two
    independent implementations must agree on the probabilities, the gradient at every materialised interface and every
    weight update."""
    c = scn.synth.CONFIGS[2]
    batch = 256
    levels, terminal = _levels(scn, 2, abi.VLEAKYRELU)
    nets = []
    for prec in (abi.PREC_AUTO, abi.PREC_FP32):
        net = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
        build_with(net, levels, terminal)
        net.set_precision(prec)
        nets.append(net)
    layers = nets[0].layers()
    weights = scn.synth.init_weights(layers, 29)
    for net in nets:
        for i, (W, B, _) in weights.items():
            net.set_weights(i, W, B, None)
    keys, off, feats = c["gen"](batch)
    labels = ((np.arange(batch) * 7) % c["nClasses"]).astype(np.int32)
    out = [net.train_batch(keys, off, feats, labels, 1e-5, 0.9) for net in nets]  # (summed gradients of 256 samples: a small rate)
    assert abi.conv_tc_take_error() == 0
    assert relerr(out[0][0], out[1][0]) < TOL
    assert out[0][1]["nll"] == pytest.approx(out[1][1]["nll"], rel=1e-4)
    checked = 0
    for i in range(len(layers) + 1):
        if i and layers[i - 1]["type"] in (0, 1):
            continue
        a, b = nets[0].dfeatures(i), nets[1].dfeatures(i)
        if b.size == 0:
            continue
        # millions of elements: a handful of near-ties fall differently in the two forwards, and each spreads over whole rows
        # of every interface below it (measured: up to 0.16 % of an interface beyond 1e-3; the top interfaces agree to 2e-6)
        assert a.size == b.size and grad_close(a, b, outliers=5e-3), "gradient of interface %d: %g" % (i, relerr(a, b))
        if i >= len(layers) - 3:
            assert relerr(a, b) < TOL, "gradient of interface %d" % i
        checked += 1
    assert checked >= 6
    for i, (W0, B0, _) in weights.items():
        (aW, aB, _), (bW, bB, _) = nets[0].get_weights(i), nets[1].get_weights(i)
        # the update is read back as w_new - w_old: what can be seen of it is bounded by the rounding of the weights themselves
        seen = lambda w0, dw: 4 * UPDATE_TOL + 2 * 6e-8 * float(np.abs(w0).max()) / max(float(np.abs(dw).max()), 1e-30)
        assert np.abs(bW - W0).max() > 100 * 6e-8 * np.abs(W0).max()
        assert relerr(aW - W0, bW - W0) < seen(W0, bW - W0), "weight update of layer %d" % i
        assert relerr(aB - B0, bB - B0) < seen(B0, bB - B0), "bias update of layer %d" % i


@pytest.mark.parametrize("cfg,batch,act", [(1, 12, "VLEAKYRELU"), (2, 8, "PRELU"), (4, 4, "PRELU"), (5, 2, "RELU")])
def test_training_steps_with_dropout_match_oracle(scn, abi, oracle, cfg, batch, act):
    """Two training steps with dropout against the oracle's restatement of the same step (fp64 accumulation), both told the
    same feature subsets, drawn here anew for each step.  Independent of the reference library: it also covers the PReLU
    layers, for which the reference has no defined result (the slopes of dropped features must stay as they are)."""
    from oracle import orc
    c = scn.synth.CONFIGS[cfg]
    levels, terminal = _levels(scn, cfg, getattr(orc, act))
    levels = [lv[:6] + (0.0 if i == 0 else 0.5,) + lv[7:] for i, lv in enumerate(levels)]
    onet = orc.OracleNet(oracle, c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    build_with(onet, levels, terminal)
    gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    build_with(gnet, levels, terminal)
    layers = gnet.layers()
    weights = scn.synth.init_weights(layers, 37)
    for i, (W, B, _) in weights.items():
        pr = np.random.default_rng(i).uniform(0.1, 0.4, len(B)).astype(np.float32) if layers[i]["act"] == orc.PRELU else None
        weights[i] = (W, B, pr)
        onet.set_weights(i, W, B, pr)
        gnet.set_weights(i, W, B, pr)
    rng = np.random.default_rng(41)
    with_dropout = [i for i, L in enumerate(layers) if L["type"] == 2 and L["dropout"] > 0]
    assert len(with_dropout) >= 2
    for step in range(2):
        subsets = {}
        for i in with_dropout:
            L = layers[i]
            keep = int(np.float32(L["nOut"]) * (np.float32(1.0) - np.float32(L["dropout"])))
            subsets[i] = np.sort(rng.choice(L["nOut"], keep, replace=False)).astype(np.int32)
            onet.set_dropout_features(i, subsets[i])
            gnet.set_dropout_features(i, subsets[i])
        keys, off, feats = c["gen"](batch, first=70 * step)
        labels = ((np.arange(batch) * 5 + step) % c["nClasses"]).astype(np.int32)
        old = {i: onet.get_weights(i) for i in weights}
        mine = {i: gnet.get_weights(i) for i in weights}
        oprobs, ostats = onet.train_step(keys, off, feats, labels, 0.01, 0.9)
        gprobs, gstats = gnet.train_batch(keys, off, feats, labels, 0.01, 0.9)
        assert abi.conv_tc_take_error() == 0
        assert relerr(gprobs, oprobs) < TOL
        assert gstats["nll"] == pytest.approx(ostats["nll"], rel=1e-4)
        assert _compare_step(gnet, onet, layers, old) >= 3
        for i in with_dropout:
            dropped = np.setdiff1d(np.arange(layers[i]["nOut"]), subsets[i])
            assert (gnet.iface_present(i + 1) == subsets[i]).all()
            assert not gnet.iface(i + 1)["features"][:, dropped].any() and not onet.iface(i + 1)["features"][:, dropped].any()
            gW, gB, gpr = gnet.get_weights(i)
            oW, oB, opr = onet.get_weights(i)
            assert (gW[:, dropped] == mine[i][0][:, dropped]).all() and (gB[dropped] == mine[i][1][dropped]).all()
            assert (oW[:, dropped] == old[i][0][:, dropped]).all() and (oB[dropped] == old[i][1][dropped]).all()
            if gpr is not None:
                assert (gpr[dropped] == mine[i][2][dropped]).all() and (gpr[subsets[i]] != mine[i][2][subsets[i]]).any()
                assert (opr[dropped] == old[i][2][dropped]).all()
