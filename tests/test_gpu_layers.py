"""GPU parity of the feature kernels through the C ABI against the oracle's CPU
restatement: integer results bit-exact, fp32 results within 1e-4 relative (the tolerance
the target states for the fp32 / 3xTF32 path), measured against the fp64-accumulating
oracle."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

RTOL_FP32 = 1e-4  # max |a-b| / max|b| over a tensor


def relerr(a, b):
    return float(np.abs(a - b).max() / max(np.abs(b).max(), 1e-30))


def random_rules(rng, rows_out, fs, rows_in, neg_frac=0.1):
    r = rng.integers(0, rows_in, size=(rows_out, fs)).astype(np.int32)
    r[rng.random(r.shape) < neg_frac] = -1
    return r


@pytest.mark.parametrize("C,sd", [(32, 4), (96, 4), (96, 8), (7, 9), (64, 27), (200, 3)])
def test_maxpool(abi, oracle, C, sd):
    rng = np.random.default_rng(C * 100 + sd)
    rows_in, rows_out = 500, 333
    feat = rng.standard_normal((rows_in, C)).astype(np.float32)
    feat[rng.random(feat.shape) < 0.2] = 0.5  # ties: the first maximum must win
    rules = random_rules(rng, rows_out, sd, rows_in, 0.2)
    rules[5, :] = -1  # a row without any usable rule
    ref_out, ref_ch = oracle.maxpool(feat, rules, sd)
    out, ch = abi.maxpool_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), sd)
    np.testing.assert_array_equal(ch.cpu().numpy(), ref_ch)
    np.testing.assert_array_equal(out.cpu().numpy(), ref_out)


def test_terminal_pool(abi, oracle):
    rng = np.random.default_rng(4)
    C, S, batch, rows_in = 96, 9, 17, 200
    feat = rng.standard_normal((rows_in, C)).astype(np.float32)
    rules = np.full((batch, S), -1, np.int32)
    for b in range(batch):
        n = rng.integers(1, S + 1)
        rules[b, :n] = rng.integers(0, rows_in, n)
    ref = oracle.terminal_pool(feat, rules, S)
    out = abi.terminal_pool_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), S)
    np.testing.assert_allclose(out.cpu().numpy(), ref, rtol=1e-6, atol=1e-6)


def test_gather(abi, oracle):
    rng = np.random.default_rng(8)
    feat = rng.standard_normal((100, 5)).astype(np.float32)
    rules = random_rules(rng, 77, 9, 100)
    ref = oracle.gather(feat, rules, 5)
    out = abi.gather_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten())
    np.testing.assert_array_equal(out.cpu().numpy(), ref)


def test_top_indices(abi, oracle):
    rng = np.random.default_rng(3)
    for n, k in ((10, 1), (10, 3), (101, 5), (2, 2), (1, 1)):
        v = rng.standard_normal((64, n)).astype(np.float32)
        v[::3] = np.round(v[::3])  # ties
        ref = np.stack([oracle.top_indices(row, k) for row in v])
        out = abi.top_indices(torch.from_numpy(v).cuda(), k)
        np.testing.assert_array_equal(out.cpu().numpy(), ref)


CONV = [
    # rows_in, rows_out, fs, nIn, N, act, p
    (300, 257, 9, 3, 32, "VLEAKYRELU", 1.0),
    (300, 100, 4, 32, 64, "VLEAKYRELU", 0.9),
    (64, 64, 1, 160, 10, "SOFTMAX", 1.0),
    (200, 513, 27, 1, 32, "RELU", 1.0),
    (128, 130, 8, 16, 96, "LEAKYRELU", 0.75),
    (50, 70, 4, 24, 40, "PRELU", 1.0),
    (50, 70, 4, 8, 33, "TANH", 1.0),
    (50, 70, 1, 8, 16, "SIGMOID", 1.0),
    (50, 70, 2, 5, 7, "NOSIGMOID", 0.5),
    # small-K kernel (K <= 64, N % 4 == 0, N > 32)
    (1000, 1357, 9, 3, 96, "VLEAKYRELU", 0.9),
    (100, 100, 1, 64, 128, "PRELU", 1.0),
    (500, 333, 27, 1, 64, "RELU", 1.0),
    (40, 41, 4, 4, 256, "LEAKYRELU", 1.0),
    # one-CTA-per-row kernel (few rows, any N) and the tile kernel (more than 2048 rows)
    (64, 64, 1, 256, 101, "SOFTMAX", 1.0),
    (90, 77, 4, 50, 101, "PRELU", 0.8),
    (400, 2500, 4, 24, 40, "VLEAKYRELU", 1.0),
    # warp-per-row kernel (N <= 32)
    (256, 256, 1, 608, 10, "SOFTMAX", 1.0),
    (90, 77, 4, 16, 20, "SOFTMAX", 0.8),
    (90, 77, 4, 16, 32, "PRELU", 0.8),
]


@pytest.mark.parametrize("rows_in,rows_out,fs,nIn,N,act,p", CONV)
def test_conv_nin_fp32(abi, oracle, rows_in, rows_out, fs, nIn, N, act, p):
    from oracle import orc
    rng = np.random.default_rng(rows_out + fs * 7 + N)
    actc = getattr(orc, act)
    K = fs * nIn
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    prelu = rng.uniform(0.1, 0.4, N).astype(np.float32) if act == "PRELU" else None
    if fs == 1:
        rows_out = rows_in
        rules = None
        X = feat
    else:
        rules = random_rules(rng, rows_out, fs, rows_in)
        X = oracle.gather(feat, rules, nIn).reshape(rows_out, K)
    ref = oracle.nin_forward(X, W, B, prelu, p, actc, accum64=True)
    out = abi.conv_nin_forward(torch.from_numpy(feat).cuda(),
                               None if rules is None else torch.from_numpy(rules).cuda().flatten(), fs,
                               torch.from_numpy(W).cuda(), torch.from_numpy(B).cuda(),
                               None if prelu is None else torch.from_numpy(prelu).cuda(), p, actc, abi.PREC_FP32)
    assert relerr(out.cpu().numpy(), ref) < RTOL_FP32


CONV_TC = [
    # rows_in, rows_out, fs, nIn, N, act, p
    (200, 300, 4, 32, 64, "VLEAKYRELU", 1.0),     # one column tile, 4 slabs
    (500, 1000, 4, 96, 192, "VLEAKYRELU", 0.9),   # the shape of the benchmark's second convolution
    (300, 257, 9, 32, 288, "RELU", 1.0),          # two column tiles of 144, ragged last row tile
    (300, 129, 8, 64, 608, "LEAKYRELU", 0.75),    # three column tiles of 208 (624 > 608: masked edge)
    (256, 256, 1, 608, 32, "NOSIGMOID", 1.0),     # plain NiN, 19 slabs
    (100, 90, 4, 128, 416, "PRELU", 1.0),
    (64, 50, 27, 32, 96, "TANH", 1.0),
    # element-wise gather (nIn not a multiple of 32; K padded to a multiple of 32)
    (1000, 1357, 9, 3, 96, "VLEAKYRELU", 0.9),    # the benchmark's first convolution, K = 27
    (200, 300, 4, 24, 64, "RELU", 1.0),
    (64, 150, 27, 1, 32, "LEAKYRELU", 1.0),
    (400, 500, 8, 4, 64, "VLEAKYRELU", 1.0),      # row-per-lane gather: four channels, K = 32 exactly
    (300, 350, 9, 2, 32, "RELU", 0.8),            # two channels, K = 18
    (100, 100, 1, 40, 48, "PRELU", 1.0),
    (300, 200, 8, 20, 288, "VLEAKYRELU", 1.0),
]


# precision -> (bound against the fp64-accumulating oracle, bound that shows the split is at work)
TC_PRECISIONS = {
    "3XTF32": (RTOL_FP32, 2e-5),   # a single tf32 product would be about 1e-3
    "SPLIT": (RTOL_FP32, 5e-5),    # bf16 operands where K >= 128 (16 bits per product), tf32 operands elsewhere
    "3XBF16": (RTOL_FP32, 5e-5),   # products carry 16 mantissa bits: about 2^-16 per product; plain bf16 is about 5e-3
    "BF16": (2e-2, 2e-2),          # the optional reduced-precision path
}


@pytest.mark.parametrize("precision", list(TC_PRECISIONS))
@pytest.mark.parametrize("rows_in,rows_out,fs,nIn,N,act,p", CONV_TC)
def test_conv_nin_tensor_core(abi, oracle, rows_in, rows_out, fs, nIn, N, act, p, precision):
    """tcgen05 with hi/lo split of both operands (kind::tf32 or bf16 under kind::f16): fp32-grade, same
    1e-4 bound as the CUDA-core kernels; plain bf16 within 2e-2."""
    from oracle import orc
    prec = getattr(abi, "PREC_" + precision)
    bound, tight = TC_PRECISIONS[precision]
    rng = np.random.default_rng(rows_out + fs * 7 + N)
    actc = getattr(orc, act)
    K = fs * nIn
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    prelu = rng.uniform(0.1, 0.4, N).astype(np.float32) if act == "PRELU" else None
    if fs == 1:
        rows_out, rules, X = rows_in, None, feat
    else:
        rules = random_rules(rng, rows_out, fs, rows_in)
        X = oracle.gather(feat, rules, nIn).reshape(rows_out, K)
    ref = oracle.nin_forward(X, W, B, prelu, p, actc, accum64=True)
    dW = torch.from_numpy(W).cuda()
    packed = abi.pack_weights(dW, prec)
    out = abi.conv_nin_forward(torch.from_numpy(feat).cuda(),
                               None if rules is None else torch.from_numpy(rules).cuda().flatten(), fs, dW,
                               torch.from_numpy(B).cuda(), None if prelu is None else torch.from_numpy(prelu).cuda(),
                               p, actc, prec, packed=packed)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    err = relerr(out.cpu().numpy(), ref)
    assert err < bound, err
    assert err < tight, err


def test_tensor_core_path_rejects_unsupported_shapes(abi):
    f = torch.zeros((4, 24), device="cuda")
    W = torch.zeros((24, 10), device="cuda")
    B = torch.zeros(10, device="cuda")
    with pytest.raises(abi.ScnError):
        abi.pack_weights(W, abi.PREC_3XTF32)  # fewer than 16 output columns
    with pytest.raises(abi.ScnError):
        abi.conv_nin_forward(f, None, 1, W, B, precision=abi.PREC_3XTF32, packed=torch.zeros(16, dtype=torch.uint8, device="cuda"))
    # AUTO falls back to the CUDA-core kernels for such shapes
    out = abi.conv_nin_forward(f, None, 1, W, B, precision=abi.PREC_AUTO)
    assert out.shape == (4, 10)


def test_conv_nin_rejects_bad_arguments(abi):
    f = torch.zeros((4, 8), device="cuda")
    W = torch.zeros((16, 16), device="cuda")
    B = torch.zeros(16, device="cuda")
    with pytest.raises(abi.ScnError):
        abi.conv_nin_forward(f, None, 2, W, B)  # fs != 1 without rules
    with pytest.raises(abi.ScnError):
        abi.conv_nin_forward(f, None, 1, W[:8].contiguous(), B, act=abi.PRELU)  # PReLU slopes missing


def test_background_rows(abi):
    keys = torch.tensor([5, -1, 7, 3, 2, -1, 9, 8, 1], dtype=torch.int32, device="cuda")
    off = torch.tensor([0, 3, 5, 5, 9], dtype=torch.int32, device="cuda")  # sample 1 has no background row, sample 2 is empty
    bg = abi.background_rows(keys, off)
    assert bg.cpu().tolist() == [1, -1, -1, 5]


@pytest.mark.parametrize("precision", ["3XTF32", "3XBF16", "SPLIT"])
def test_split_k_matches_single_pass(abi, oracle, precision):
    """Layers with few output tiles split K over several CTAs; the partial sums are added in a
    fixed order, so repeated runs are bit-identical; split and unsplit kernels differ only by
    the accumulation order (K = 2048 here) and both stay within the 1e-4 bound of the oracle."""
    rng = np.random.default_rng(12)
    rows, K, N = 200, 2048, 96
    feat = torch.from_numpy(rng.standard_normal((rows, K)).astype(np.float32)).cuda()
    W = torch.from_numpy((rng.standard_normal((K, N)) * 0.02).astype(np.float32)).cuda()
    B = torch.zeros(N, device="cuda")
    prec = getattr(abi, "PREC_" + precision)
    packed = abi.pack_weights(W, prec)
    assert abi.lib().scn_conv_nin_workspace_bytes(rows, 1, K, N, prec) > 0
    a = abi.conv_nin_forward(feat, None, 1, W, B, precision=prec, packed=packed, split_k=True)
    b = abi.conv_nin_forward(feat, None, 1, W, B, precision=prec, packed=packed, split_k=True)
    c = abi.conv_nin_forward(feat, None, 1, W, B, precision=prec, packed=packed, split_k=False)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    assert torch.equal(a, b)
    assert relerr(a.cpu().numpy(), c.cpu().numpy()) < 5e-5
    ref = oracle.nin_forward(feat.cpu().numpy(), W.cpu().numpy(), B.cpu().numpy(), accum64=True)
    assert relerr(a.cpu().numpy(), ref) < RTOL_FP32
    assert relerr(c.cpu().numpy(), ref) < RTOL_FP32


def test_conv_nin_with_row_count_on_the_device(abi, oracle):
    """scn_conv_nin_forward_dyn: buffers sized for an upper bound, the kernel reads the real row count from
    device memory (how the first layer starts before the rulebook counts reach the host)."""
    from oracle import orc
    rng = np.random.default_rng(21)
    rows_in, bound, rows, fs, nIn, N = 700, 1000, 777, 9, 3, 96
    K = fs * nIn
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    rules = random_rules(rng, bound, fs, rows_in)
    X = oracle.gather(feat, rules[:rows], nIn).reshape(rows, K)
    ref = oracle.nin_forward(X, W, B, None, 0.9, orc.VLEAKYRELU, accum64=True)
    dW = torch.from_numpy(W).cuda()
    packed = abi.pack_weights(dW, abi.PREC_3XTF32)
    d_rows = torch.tensor([rows, 0, 0, 0], dtype=torch.int32, device="cuda")
    out = abi.conv_nin_forward_dyn(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), fs, dW, torch.from_numpy(B).cuda(),
                                   d_rows, bound, None, 0.9, abi.VLEAKYRELU, packed)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    out = out.cpu().numpy()
    assert relerr(out[:rows], ref) < RTOL_FP32
    assert not out[rows:].any()  # rows past the count are not written
    # a count above the bound is clamped
    d_rows[0] = bound + 500
    out2 = abi.conv_nin_forward_dyn(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), fs, dW, torch.from_numpy(B).cuda(),
                                    d_rows, bound, None, 0.9, abi.VLEAKYRELU, packed)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0 and np.isfinite(out2.cpu().numpy()).all()


@pytest.mark.parametrize("rows_in,windows,fs,nIn,N,cells,act", [
    (600, 333, 4, 32, 64, 4, "VLEAKYRELU"),     # ragged last tile, A from tensor memory
    (1200, 700, 9, 3, 96, 4, "VLEAKYRELU"),     # the benchmark's first convolution + pooling (element-wise gather)
    (500, 150, 4, 96, 192, 4, "RELU"),
    (300, 90, 8, 32, 288, 8, "LEAKYRELU"),      # 2^3 windows, two column tiles
    (200, 70, 4, 64, 32, 2, "PRELU"),
    (800, 260, 27, 1, 32, 8, "VLEAKYRELU"),     # a 3-D first layer (one channel, 3^3 filter) + 2^3 pooling: row-per-lane gather, two epilogue groups
    (500, 200, 8, 4, 48, 2, "RELU"),
])
@pytest.mark.parametrize("precision", ["3XTF32", "SPLIT"])
def test_conv_nin_maxpool_fused(abi, oracle, rows_in, windows, fs, nIn, N, cells, act, precision):
    _fused_case(abi, oracle, rows_in, windows, fs, nIn, N, cells, act, False, getattr(abi, "PREC_" + precision))


@pytest.mark.parametrize("rows_in,windows,fs,nIn,N,cells,act", [
    (300, 60, 4, 256, 128, 4, "VLEAKYRELU"),    # two tiles, 32 slabs: K is split and the pooling runs in the finishing kernel
    (200, 30, 8, 128, 608, 8, "RELU"),
])
@pytest.mark.parametrize("precision", ["3XTF32", "SPLIT"])
def test_conv_nin_maxpool_with_k_split(abi, oracle, rows_in, windows, fs, nIn, N, cells, act, precision):
    prec = getattr(abi, "PREC_" + precision)
    assert abi.lib().scn_conv_nin_workspace_bytes(windows * cells + 5, fs, nIn, N, prec) > 0
    _fused_case(abi, oracle, rows_in, windows, fs, nIn, N, cells, act, True, prec)


def _fused_case(abi, oracle, rows_in, windows, fs, nIn, N, cells, act, split, prec):
    """Gather + NiN + non-overlapping max pooling in one kernel against the oracle's three steps: pooled values
    within the fp32 tolerance, every choice names an input whose value is the window's maximum."""
    from oracle import orc
    rng = np.random.default_rng(windows + N)
    actc = getattr(orc, act)
    K = fs * nIn
    rows_mid = windows * cells + 5  # rows of the learnt layer's output (a few are in no window)
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    prelu = rng.uniform(0.1, 0.4, N).astype(np.float32) if act == "PRELU" else None
    rules = random_rules(rng, rows_mid, fs, rows_in)
    pool = rng.permutation(rows_mid)[: windows * cells].astype(np.int32).reshape(windows, cells)
    pool[rng.random(pool.shape) < 0.15] = -1      # cells without an input
    pool[3] = -1                                   # a window with none at all
    pool[5, :] = 7                                 # the same row several times: the first wins
    X = oracle.gather(feat, rules, nIn).reshape(rows_mid, K)
    mid = oracle.nin_forward(X, W, B, prelu, 0.9, actc, accum64=True)
    ref_v, ref_c = oracle.maxpool(mid.astype(np.float32), pool, cells)
    dW = torch.from_numpy(W).cuda()
    packed = abi.pack_weights(dW, prec)
    out, ch = abi.conv_nin_maxpool_forward(torch.from_numpy(feat).cuda(), torch.from_numpy(rules).cuda().flatten(), fs, dW,
                                           torch.from_numpy(B).cuda(), torch.from_numpy(pool).cuda().flatten(), cells,
                                           None if prelu is None else torch.from_numpy(prelu).cuda(), 0.9, actc, packed,
                                           rows_unpooled=rows_mid if split else 0, split_k=split, precision=prec)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    out, ch = out.cpu().numpy(), ch.cpu().numpy()
    assert relerr(out, ref_v) < RTOL_FP32
    assert (ch[3] == -1).all() and not out[3].any()
    ok = ch >= 0
    assert (ok == (ref_c >= 0)).all()
    picked = mid.reshape(-1)[ch[ok]]
    assert np.abs(picked - ref_v[ok]).max() <= 1e-4 * np.abs(ref_v).max()  # a choice may differ from the oracle's only between near-equal values
    rows_of = ch[ok] // N
    assert (ch[ok] % N == np.broadcast_to(np.arange(N), ch.shape)[ok]).all()
    assert np.isin(rows_of, pool[pool >= 0]).all()
    assert (ch[5] == pool[5, 0] * N + np.arange(N)).all()


@pytest.mark.parametrize("rows_in,rows,fs,nIn,N,N2,act,act2", [
    (1024, 256, 4, 512, 608, 10, "VLEAKYRELU", "SOFTMAX"),   # the top of the benchmark network: last convolution + classifier
    (300, 100, 1, 1024, 96, 16, "RELU", "NOSIGMOID"),        # plain learnt layers, no rules
    (200, 40, 8, 128, 288, 3, "LEAKYRELU", "SOFTMAX"),
])
@pytest.mark.parametrize("precision", ["3XTF32", "SPLIT"])
def test_conv_nin_then_small_nin(abi, oracle, rows_in, rows, fs, nIn, N, N2, act, act2, precision):
    """A learnt layer that splits K and the small learnt layer behind it in one call (the second applied by the kernel
    that adds the partial sums) against the oracle's two layers: both outputs within the fp32 tolerance."""
    from oracle import orc
    rng = np.random.default_rng(rows + N2)
    K = fs * nIn
    feat = rng.standard_normal((rows_in, nIn)).astype(np.float32)
    W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
    B = (rng.standard_normal(N) * 0.1).astype(np.float32)
    W2 = (rng.standard_normal((N, N2)) * np.sqrt(2.0 / N)).astype(np.float32)
    B2 = (rng.standard_normal(N2) * 0.1).astype(np.float32)
    if fs > 1:
        rules = random_rules(rng, rows, fs, rows_in)
        X = oracle.gather(feat, rules, nIn).reshape(rows, K)
        d_rules = torch.from_numpy(rules).cuda().flatten()
    else:
        feat = feat[:rows]
        X, d_rules = feat, None
    mid_ref = oracle.nin_forward(X, W, B, None, 0.9, getattr(orc, act), accum64=True)
    out_ref = oracle.nin_forward(mid_ref.astype(np.float32), W2, B2, None, 1.0, getattr(orc, act2), accum64=True)
    dW = torch.from_numpy(W).cuda()
    prec = getattr(abi, "PREC_" + precision)
    packed = abi.pack_weights(dW, prec)
    assert abi.lib().scn_conv_nin_workspace_bytes(rows, fs, nIn, N, prec) > 0
    mid, out = abi.conv_nin_nin_forward(torch.from_numpy(feat).cuda(), d_rules, fs, dW, torch.from_numpy(B).cuda(), torch.from_numpy(W2).cuda(),
                                        torch.from_numpy(B2).cuda(), None, 0.9, getattr(abi, act), 1.0, getattr(abi, act2), packed, precision=prec)
    torch.cuda.synchronize()
    assert abi.conv_tc_take_error() == 0
    assert relerr(mid.cpu().numpy(), mid_ref) < RTOL_FP32
    assert relerr(out.cpu().numpy(), out_ref) < RTOL_FP32


def test_classifier_result_block(abi, oracle):
    """scn_classifier_result: the probabilities, the nTop classes of every row (vectorTopIndices order) and the
    tensor-core error word as one block; the word is zero as long as no kernel gave up a wait."""
    rng = np.random.default_rng(31)
    for rows, n, k in ((256, 10, 1), (64, 101, 5), (3, 20, 3), (1, 2, 2)):
        v = rng.random((rows, n)).astype(np.float32)
        v[::3] = np.round(v[::3], 1)  # ties
        p, t, flag = abi.classifier_result(torch.from_numpy(v).cuda(), k)
        np.testing.assert_array_equal(p.numpy(), v)
        np.testing.assert_array_equal(t.numpy(), np.stack([oracle.top_indices(row, k) for row in v]))
        assert flag == 0
    assert abi.lib().scn_conv_tc_error_word() != 0


@pytest.mark.parametrize("trans_a,trans_b", [(False, False), (True, False), (False, True), (True, True)])
@pytest.mark.parametrize("l,m,r", [(70, 45, 33), (128, 64, 64), (1, 300, 5), (257, 1, 130)])
def test_sgemm_rowmajor_forms(abi, trans_a, trans_b, l, m, r):
    """The four products of the reference's cuBLAS wrappers (utilities.cu:132-169: AB, AtB, ABt, AtBt on row-major
    matrices with alpha and beta) against float64 numpy; with beta = 0 the old contents of C are not read."""
    import torch
    rng = np.random.default_rng(l * 1000 + m * 10 + r)
    A = rng.standard_normal((l, m))
    B = rng.standard_normal((m, r))
    C0 = rng.standard_normal((l, r))
    dA = torch.from_numpy(np.ascontiguousarray(A.T if trans_a else A, np.float32)).cuda()
    dB = torch.from_numpy(np.ascontiguousarray(B.T if trans_b else B, np.float32)).cuda()
    dC = torch.from_numpy(C0.astype(np.float32)).cuda()
    abi.sgemm_rowmajor(dA, dB, dC, l, m, r, 0.7, 0.3, trans_a, trans_b)
    want = 0.7 * (A.astype(np.float32).astype(np.float64) @ B.astype(np.float32).astype(np.float64)) + 0.3 * C0.astype(np.float32)
    assert relerr(dC.cpu().numpy(), want) < 1e-5
    dC = torch.full((l, r), float("nan"), dtype=torch.float32).cuda()
    abi.sgemm_rowmajor(dA, dB, dC, l, m, r, 1.0, 0.0, trans_a, trans_b)
    assert relerr(dC.cpu().numpy(), want / 0.7 - 0.3 / 0.7 * C0.astype(np.float32)) < 1e-5
