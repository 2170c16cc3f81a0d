"""Index learning (IndexLearnerLayer.h; SparseConvNetCUDA.cu:211-225, 443-474): every picture of the training set is its
own class, a batch works on the columns of its own pictures only.  The product's steps against the reference's own
processIndexLearnerBatch (compiled test-only, oracle/_ref_gpu) on the batches the reference's BatchProducer drew."""
import numpy as np
import pytest

from netutil import relerr

pytestmark = pytest.mark.gpu

TOL = 1e-4
UPDATE_TOL = 5e-3
PICTURES, BATCH, N_IN = 10, 4, 3


def _build(net, act, dropout):
    net.addLeNetLayerMP(32, 3, 1, 2, 2, act, 0.0, 1)
    net.addLeNetLayerMP(64, 2, 1, 2, 2, act, dropout, 1)
    net.addLeNetLayerMP(96, 2, 1, 1, 1, act, 0.0, 1)
    net.addIndexLearnerLayer()


def _pictures(S, seed):
    rng = np.random.default_rng(seed)
    keys, feats, off = [], [], [0]
    for _ in range(PICTURES):
        k = np.unique(rng.integers(0, S * S, 4 * S))
        keys.append(np.concatenate([[-1], k]))
        feats.append(np.concatenate([np.zeros((1, N_IN)), rng.uniform(-1, 1, (len(k), N_IN))]))
        off.append(off[-1] + len(k) + 1)
    return np.concatenate(keys).astype(np.int32), np.array(off, np.int32), np.concatenate(feats).astype(np.float32)


@pytest.mark.parametrize("dropout", [0.0, 0.5])
def test_index_learning_steps_match_the_reference(scn, abi, tmp_path, dropout):
    from oracle import orc
    if not orc.ReferenceGPU.available():
        pytest.skip("oracle/_ref_gpu/libscn_ref_gpu.so not built")
    gnet = scn.net.Net(2, N_IN, PICTURES, 1, 0)
    _build(gnet, abi.VLEAKYRELU, dropout)
    ref = orc.ReferenceGPU(2, N_IN, PICTURES, 1, 0)
    _build(ref, orc.VLEAKYRELU, dropout)
    layers = gnet.layers()
    assert layers[-1]["type"] == 7 and layers[-1]["nOut"] == PICTURES and gnet.inputSpatialSize == ref.inputSpatialSize
    learnt = [i for i, L in enumerate(layers) if L["type"] == 2]
    for i, (W, B, _) in scn.synth.init_weights(layers, 31).items():
        gnet.set_weights(i, W, B, None)
    base = str(tmp_path / "x")
    gnet.save_weights(base, 0)  # (the index learner's zero weights included)
    ref.load_weights(base, 0)
    ref.seed_dropout(77)
    top = len(layers) - 1
    assert not gnet.get_weights(top)[0].any()
    keys, off, feats = _pictures(gnet.inputSpatialSize, 5)
    lr, mom = 0.01, 0.9
    seen = set()
    for step in range(4):
        before = {i: gnet.get_weights(i) for i in learnt + [top]}
        rbefore = {i: ref.layer_weights(i) for i in learnt + [top]}
        nums, rprobs, rstats = ref.index_learner_batch(keys, off, feats, BATCH, lr, mom)
        assert len(nums) == BATCH and len(set(nums.tolist())) == BATCH
        met_before = bool(seen & set(nums.tolist()))  # a picture whose column has been trained: only then is there a gradient below
        seen.update(nums.tolist())
        for i in learnt:  # the feature subsets the reference drew (layers with dropout)
            present = ref.iface(i + 1)["present"]
            gnet.set_dropout_features(i, present if len(present) < layers[i]["nOut"] else [])
        k2 = np.concatenate([keys[off[s]:off[s + 1]] for s in nums])
        f2 = np.concatenate([feats[off[s]:off[s + 1]] for s in nums])
        o2 = np.concatenate([[0], np.cumsum([off[s + 1] - off[s] for s in nums])]).astype(np.int32)
        gprobs, gstats = gnet.index_learner_batch(k2, o2, f2, nums, lr, mom)
        assert abi.conv_tc_take_error() == 0
        assert relerr(gprobs, rprobs) < TOL
        assert gstats["nll"] == pytest.approx(rstats["nll"], rel=1e-4)
        assert gstats["mistakes"] == rstats["mistakes"]
        # the index learner: only the batch's columns move, and they move alike
        W0, rW0 = before[top][0], rbefore[top][0]
        gW, rW = gnet.get_weights(top)[0], ref.layer_weights(top)[0]
        others = np.setdiff1d(np.arange(PICTURES), nums)
        assert (gW[:, others] == W0[:, others]).all() and (rW[:, others] == rW0[:, others]).all()
        assert np.abs(rW - rW0).max() > 0
        assert relerr((gW - W0)[:, nums], (rW - rW0)[:, nums]) < UPDATE_TOL
        for i in learnt:
            gWi, rWi = gnet.get_weights(i)[0], ref.layer_weights(i)[0]
            if met_before:
                assert np.abs(rWi - rbefore[i][0]).max() > 0
                assert relerr(gWi - before[i][0], rWi - rbefore[i][0]) < 4 * UPDATE_TOL, "weight update of layer %d" % i
            else:  # the batch's columns of the index learner are still zero: nothing flows back, nothing moves
                assert (gWi == before[i][0]).all() and (rWi == rbefore[i][0]).all()
    assert len(seen) > BATCH
    # the weight file carries the index learner's weights: the reference reads the product's file back
    gnet.save_weights(base, 1)
    ref.load_weights(base, 1)
    np.testing.assert_array_equal(ref.layer_weights(top)[0], gnet.get_weights(top)[0])
