"""The result exchange between the GPUs of one node (peer stores + bounded waits, csrc/exchange.cu).

On one GPU the ranks are emulated in one process: every rank has its own buffer, all publishes of a step are enqueued
before any collect of it, so no kernel ever waits for another launch.  The time limit is tested with a step that one rank
never publishes (the collector returns with that rank's bit set; nothing faults or hangs).  With two or more GPUs a
second test runs real ranks as processes, the buffers mapped through CUDA IPC."""
import os
import socket
import sys

import numpy as np
import pytest
import torch

from netutil import make_pair

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("world,cap_rows,nC", [(1, 5, 10), (3, 7, 10), (8, 256, 10), (16, 33, 3)])
def test_publish_then_collect_round_trips_every_block(abi, world, cap_rows, nC):
    cap = cap_rows * nC
    bufs = [abi.ExchangeBuffer(world, cap) for _ in range(world)]
    peers = [b.ptr for b in bufs]
    g = torch.Generator(device="cuda").manual_seed(3)
    try:
        for step in range(1, 11):  # more steps than slots: every slot is reused
            rows = [(step * 5 + r * 3) % (cap_rows + 1) for r in range(world)]
            blocks = [torch.rand((rows[r], nC), device="cuda", generator=g) + step for r in range(world)]
            for r in range(world):
                abi.exchange_publish(blocks[r].reshape(-1), rows[r], peers, r, cap, step)
            for r in range(world):
                out, got_rows, status = abi.exchange_collect(peers[r], world, cap, step)
                assert int(status.item()) == 0
                assert got_rows.tolist() == rows
                for s in range(world):
                    torch.testing.assert_close(out[s, : rows[s] * nC], blocks[s].reshape(-1), rtol=0, atol=0)
    finally:
        torch.cuda.synchronize()
        for b in bufs:
            b.free()


def test_a_rank_that_never_publishes_is_reported_not_waited_for(abi):
    world, cap = 3, 40
    bufs = [abi.ExchangeBuffer(world, cap) for _ in range(world)]
    peers = [b.ptr for b in bufs]
    abi.exchange_set_timeout_ms(50)
    try:
        blk = torch.arange(40, dtype=torch.float32, device="cuda")
        abi.exchange_publish(blk, 4, peers, 0, cap, 1)
        abi.exchange_publish(blk + 100, 4, peers, 2, cap, 1)  # rank 1 stays silent
        out, rows, status = abi.exchange_collect(peers[0], world, cap, 1)
        torch.cuda.synchronize()
        assert int(status.item()) == 1 << 1
        assert rows.tolist() == [4, -1, 4]
        torch.testing.assert_close(out[0], blk, rtol=0, atol=0)
        torch.testing.assert_close(out[2], blk + 100, rtol=0, atol=0)
        assert float(out[1].abs().max()) == 0.0
        # the context is still usable and the late rank can still deliver
        abi.exchange_publish(blk + 7, 4, peers, 1, cap, 1)
        out, rows, status = abi.exchange_collect(peers[0], world, cap, 1)
        assert int(status.item()) == 0 and rows.tolist() == [4, 4, 4]
    finally:
        abi.exchange_set_timeout_ms(2000)
        torch.cuda.synchronize()
        for b in bufs:
            b.free()


def test_bad_arguments_are_refused(abi):
    assert abi.lib().scn_exchange_buffer_bytes(17, 10) == 0
    b = abi.ExchangeBuffer(2, 8)
    try:
        blk = torch.zeros(9, device="cuda")
        with pytest.raises(abi.ScnError):
            abi.exchange_publish(blk, 1, [b.ptr, b.ptr], 0, 8, 1)  # more floats than the buffer was made for
        with pytest.raises(abi.ScnError):
            abi.exchange_publish(blk[:8], 1, [b.ptr, b.ptr], 0, 8, 0)  # steps count from 1
        with pytest.raises(abi.ScnError):
            abi.exchange_publish(blk[:8], 1, [b.ptr, b.ptr], 2, 8, 1)  # rank outside the group
    finally:
        b.free()


def test_sharded_forward_delivers_every_ranks_results_one_step_later(scn, abi, oracle):
    """Three emulated ranks, each a network of its own on a third of the batch: what forward_host_exchange hands out as
    the step before equals the ranks' own results of that step; flush returns the last step."""
    cfg, world, per = 2, 3, 8
    c = scn.synth.CONFIGS[cfg]
    nets = [make_pair(scn, oracle, cfg)[0] for _ in range(world)]
    for r, n in enumerate(nets):
        n.exchange_create(world, r, per)
    bufs = [n.exchange_buffer() for n in nets]
    for n in nets:
        n.exchange_connect_local(bufs)
    prev = None
    for step in range(5):
        own = []
        for r, n in enumerate(nets):
            rows = per - (step + r) % 3  # ragged blocks
            keys, off, feats = c["gen"](rows, first=(step * world + r) * per)
            plain, plain_top = n.forward_host(keys, off, feats)
            probs, top, gathered, grows = n.forward_host_exchange(keys, off, feats)
            np.testing.assert_array_equal(probs, plain)
            np.testing.assert_array_equal(top, plain_top)
            own.append(probs)
            if prev is None:
                assert grows.tolist() == [-1] * world
            else:
                assert grows.tolist() == [len(p) for p in prev]
                for s in range(world):
                    np.testing.assert_array_equal(gathered[s, : len(prev[s])], prev[s])
        prev = own
    for n in nets:
        gathered, grows = n.exchange_flush()
        assert grows.tolist() == [len(p) for p in prev]
        for s in range(world):
            np.testing.assert_array_equal(gathered[s, : len(prev[s])], prev[s])
    assert abi.conv_tc_take_error() == 0
    with pytest.raises(scn.abi.ScnError):  # more samples than the exchange was made for
        keys, off, feats = c["gen"](per + 1)
        nets[0].forward_host_exchange(keys, off, feats)
    torch.cuda.synchronize()
    for n in nets:
        n.exchange_destroy()


def test_two_halves_entry_point_with_exchange(scn, abi, oracle):
    """forward_host_begin / forward_host_end(exchange=True) on two emulated ranks: uploads one batch ahead, results of the
    other rank one step later."""
    cfg, world, per = 2, 2, 5
    c = scn.synth.CONFIGS[cfg]
    nets = [make_pair(scn, oracle, cfg)[0] for _ in range(world)]
    for r, n in enumerate(nets):
        n.exchange_create(world, r, per)
    bufs = [n.exchange_buffer() for n in nets]
    for n in nets:
        n.exchange_connect_local(bufs)
    steps = 4
    data = [[c["gen"](per - (s + r) % 2, first=(s * world + r) * per) for s in range(steps)] for r in range(world)]
    want = [[nets[r].forward_host(*data[r][s])[0] for s in range(steps)] for r in range(world)]
    for r in range(world):
        nets[r].forward_host_begin(*data[r][0])
    for s in range(steps):
        for r in range(world):
            if s + 1 < steps:
                nets[r].forward_host_begin(*data[r][s + 1])
            probs, _, gathered, rows = nets[r].forward_host_end(True)
            np.testing.assert_array_equal(probs, want[r][s])
            if s == 0:
                assert rows.tolist() == [-1] * world
            else:
                assert rows.tolist() == [len(want[q][s - 1]) for q in range(world)]
                for q in range(world):
                    np.testing.assert_array_equal(gathered[q, : rows[q]], want[q][s - 1])
    for r in range(world):
        gathered, rows = nets[r].exchange_flush()
        for q in range(world):
            np.testing.assert_array_equal(gathered[q, : rows[q]], want[q][steps - 1])
    torch.cuda.synchronize()
    for n in nets:
        n.exchange_destroy()


def test_device_resident_steps_deliver_one_step_later(scn, abi, oracle):
    """The device-resident form (exchange kernel beside the network's stream): two emulated ranks, three steps and the
    collect-only call that ends the run."""
    cfg, world, per = 2, 2, 6
    c = scn.synth.CONFIGS[cfg]
    nC = c["nClasses"]
    nets = [make_pair(scn, oracle, cfg)[0] for _ in range(world)]
    for r, n in enumerate(nets):
        n.exchange_create(world, r, per)
    bufs = [n.exchange_buffer() for n in nets]
    for n in nets:
        n.exchange_connect_local(bufs)
    dev = torch.device("cuda")
    gathered = [[torch.zeros((world, per, nC), device=dev) for _ in range(2)] for _ in range(world)]
    status = [torch.zeros(world + 1, dtype=torch.int32, device=dev) for _ in range(world)]
    d_top = torch.empty((per, 1), dtype=torch.int32, device=dev)
    history = []
    for step in range(3):
        own = []
        for r, n in enumerate(nets):
            keys, off, feats = c["gen"](per, first=(step * world + r) * per)
            want, _ = n.forward_host(keys, off, feats)
            dk, do, df = (torch.from_numpy(x).to(dev) for x in (keys, off, feats))
            db = do[:-1].clone()
            d_probs = torch.empty((per, nC), device=dev)
            n.forward_device(dk, do, db, df, int(np.diff(off).max() - 1), d_probs, d_top)
            n.exchange_step_device(d_probs, per, gathered[r][(step - 1) & 1], status[r])
            torch.cuda.synchronize()  # (the emulated ranks share one GPU: a step is published before the next rank collects)
            np.testing.assert_array_equal(d_probs.cpu().numpy(), want)
            own.append(want)
        history.append(own)
    for r, n in enumerate(nets):
        n.exchange_step_device(None, 0, gathered[r][2 & 1], status[r])
    torch.cuda.synchronize()
    for r in range(world):
        assert int(status[r][world].item()) == 0
        assert status[r][:world].tolist() == [per] * world
        for s_ in range(world):
            np.testing.assert_array_equal(gathered[r][0][s_].cpu().numpy(), history[2][s_])  # step 2, collected last
            np.testing.assert_array_equal(gathered[r][1][s_].cpu().numpy(), history[1][s_])  # step 1, collected in step 2
    for n in nets:
        n.exchange_destroy()


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _rank_process(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import importlib
    import torch.distributed as dist
    scn = importlib.import_module("sparseconvnet-archived_b200")
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg, per = 1, 6
        c = scn.synth.CONFIGS[cfg]
        net = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
        scn.synth.build_network(net, cfg)
        for i, (W, B, pr) in scn.synth.init_weights(net.layers()).items():
            net.set_weights(i, W, B, pr)
        assert scn.shard.connect_exchange(net, per)
        record = []
        for step in range(6):
            keys, off, feats = c["gen"](per - (step + rank) % 2, first=(step * world + rank) * per)
            probs, _, gathered, rows = net.forward_host_exchange(keys, off, feats)
            record.append((probs, gathered.copy(), rows.copy()))
        gathered, rows = net.exchange_flush()
        record.append((None, gathered.copy(), rows.copy()))
        scn.shard.disconnect_exchange(net)
        np.save(os.path.join(out_dir, "rank%d.npy" % rank), np.array(record, dtype=object), allow_pickle=True)
    finally:
        dist.destroy_process_group()


def test_two_processes_on_two_gpus(abi, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mp.spawn(_rank_process, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    rec = [np.load(str(tmp_path / ("rank%d.npy" % r)), allow_pickle=True) for r in range(world)]
    for r in range(world):
        assert rec[r][0][2].tolist() == [-1] * world
        for step in range(1, 7):
            gathered, rows = rec[r][step][1], rec[r][step][2]
            for s in range(world):
                want = rec[s][step - 1][0]
                assert rows[s] == len(want)
                np.testing.assert_array_equal(gathered[s, : len(want)], want)
