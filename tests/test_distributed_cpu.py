"""The N > 1 path on CPU: two gloo ranks each run the forward of their shard of a batch (the
CPU oracle stands in for the per-rank GPU forward) and all-gather the probabilities; the
result must equal the single-process forward of the whole batch.  This is the property the
multi-GPU benchmark relies on: sharding by sample needs no data-path collective."""
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, cfg, n, balanced, out_path):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    scn = importlib.import_module("sparseconvnet-archived_b200")
    from oracle import orc
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        c = scn.synth.CONFIGS[cfg]
        onet = orc.OracleNet(orc.Oracle(), c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
        scn.synth.build_network(onet, cfg)
        for i, (W, B, pr) in scn.synth.init_weights(onet.layers()).items():
            onet.set_weights(i, W, B, pr)
        keys, off, feats = c["gen"](n)
        if balanced:
            bounds = scn.shard.balanced_ranges(np.diff(off) - 1, world)
            lo, hi = bounds[rank], bounds[rank + 1]
            counts = [bounds[r + 1] - bounds[r] for r in range(world)]
        else:
            lo, hi = scn.shard.shard_range(n, rank, world)
            counts = [scn.shard.shard_range(n, r, world)[1] - scn.shard.shard_range(n, r, world)[0] for r in range(world)]
        k, o, f = scn.shard.take_samples(keys, off, feats, lo, hi)
        probs, _ = onet.forward(k.astype(np.int64), o, f)
        local = torch.from_numpy(probs)
        if len(set(counts)) == 1:
            full = scn.shard.gather_probabilities(local)
        else:
            full = scn.shard.gather_ragged(local, counts)
        if rank == 0:
            whole, _ = onet.forward(keys.astype(np.int64), off, feats)
            np.save(out_path, np.stack([full.numpy(), whole]))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("cfg,n,balanced", [(1, 6, False), (1, 7, False), (3, 4, True)])
def test_two_ranks_equal_one(tmp_path, scn, oracle, cfg, n, balanced):
    out = str(tmp_path / "res.npy")
    mp.spawn(_worker, args=(2, _free_port(), cfg, n, balanced, out), nprocs=2, join=True)
    full, whole = np.load(out)
    np.testing.assert_array_equal(full, whole)  # same arithmetic per sample: bit-identical


def test_shard_helpers(scn):
    sh = scn.shard
    assert [sh.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    assert sh.shard_range(256, 7, 8) == (224, 256)
    b = sh.balanced_ranges([10, 10, 10, 10, 40, 40], 2)
    assert b[0] == 0 and b[-1] == 6 and b[1] in (4, 5)
    b = sh.balanced_ranges([5] * 8, 8)
    assert b == list(range(9))
    keys = np.array([-1, 3, 4, -1, 7], np.int32)
    off = np.array([0, 3, 5], np.int32)
    feats = np.arange(10, dtype=np.float32).reshape(5, 2)
    k, o, f = sh.take_samples(keys, off, feats, 1, 2)
    assert k.tolist() == [-1, 7] and o.tolist() == [0, 2] and f.tolist() == [[6, 7], [8, 9]]
