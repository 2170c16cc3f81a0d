"""Sharding by sample on the GPU: a batch cut into contiguous blocks of samples (equal counts, or equal numbers of
active sites for ragged samples), every block run through the product on its own, gives the whole batch's result.

Rulebooks and grids of a block are the whole batch's with the block's first row subtracted (bit-exact); pooled
features and probabilities agree within 1e-5 of the largest (a block has fewer rows than the batch, so a layer may
split K differently and add its partial sums in another order); top-1 is equal.  One GPU runs the blocks one after
the other: this is what each rank of `bench.py --gpus N` does with its block."""
import numpy as np
import pytest

from netutil import make_pair, relerr

pytestmark = pytest.mark.gpu

TOL = 1e-5


def _blocks(scn, off, world, balanced):
    n = len(off) - 1
    if balanced:
        return scn.shard.balanced_ranges(np.diff(off) - 1, world)
    return [scn.shard.shard_range(n, r, world)[0] for r in range(world)] + [n]


@pytest.mark.parametrize("cfg,n,world,balanced", [(2, 64, 2, False), (2, 33, 4, False), (1, 24, 3, True), (3, 12, 2, True),
                                                  (3, 12, 3, True), (4, 16, 2, True), (5, 3, 2, True)])
def test_blocks_of_samples_equal_the_whole_batch(scn, abi, oracle, cfg, n, world, balanced):
    c = scn.synth.CONFIGS[cfg]
    gnet, _ = make_pair(scn, oracle, cfg)
    keys, off, feats = c["gen"](n)
    whole_probs, whole_top = gnet.forward_host(keys, off, feats)
    layers = gnet.layers()
    whole = [gnet.iface(i, features=(i > 0 and layers[i - 1]["type"] in (3, 4, 5))) for i in range(len(layers) + 1)]
    bounds = _blocks(scn, off, world, balanced)
    assert bounds[0] == 0 and bounds[-1] == n and all(a <= b for a, b in zip(bounds, bounds[1:]))
    if balanced:  # no block is heavier than an equal share of the sites plus one sample
        sites = np.diff(off) - 1
        heaviest = max(int(sites[a:b].sum()) for a, b in zip(bounds, bounds[1:]))
        assert heaviest <= sites.sum() / world + sites.max()
    probs, tops = [], []
    row0 = [0] * (len(layers) + 1)
    for lo, hi in zip(bounds, bounds[1:]):
        if lo == hi:
            continue
        k, o, f = scn.shard.take_samples(keys, off, feats, lo, hi)
        p, t = gnet.forward_host(k, o, f)
        assert abi.conv_tc_take_error() == 0
        probs.append(p)
        tops.append(t)
        base = list(row0)  # this block's first row at every interface of the whole batch
        for i in range(len(layers) + 1):
            feat = i > 0 and layers[i - 1]["type"] in (3, 4, 5)
            g, w = gnet.iface(i, features=feat), whole[i]
            rows = g["nSpatialSites"]
            np.testing.assert_array_equal(g["row_keys"], w["row_keys"][base[i]:base[i] + rows], err_msg="grid of interface %d" % i)
            if i and g["rules"].size:
                cells = g["rules"].size // max(rows, 1)
                wr = w["rules"].reshape(-1, cells)[base[i]:base[i] + rows]
                gr = g["rules"].reshape(-1, cells)
                shifted = np.where(gr >= 0, gr + base[i - 1], gr)
                np.testing.assert_array_equal(shifted, wr, err_msg="rulebook of interface %d" % i)
            if feat and rows:
                wf = w["features"][base[i]:base[i] + rows]
                assert relerr(g["features"], wf) < TOL, i
            row0[i] += rows
    for i in range(len(layers) + 1):
        assert row0[i] == whole[i]["nSpatialSites"], i
    assert relerr(np.concatenate(probs), whole_probs) < TOL
    np.testing.assert_array_equal(np.concatenate(tops), whole_top)
