#!/usr/bin/env python
"""Benchmark of the forward hot path: samples/sec of a DeepCNet(5,100)-style network
(addLeNetLayerMP levels with conv + 2/2 max pooling, builder-rounded widths 96..608) on the
CIFAR-10-shaped dense-in-sparse 2-D workload, batch 256 per GPU.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

One "step" = one full forward of one batch: rule construction for every layer on the
device, all fused conv/NiN, pooling and softmax kernels, top-1, and (N > 1) the all-gather
of the class probabilities (over peer memory, inside the forward call).  Rank r of N processes
its own 256 samples (weak scaling).

  value     device-timed throughput with the inputs already resident in HBM
  e2e       the same through the host-buffer entry points (scn_net_forward_host_begin / _end:
            the upload of batch j + 1 runs while batch j is computed, as the reference's
            producer threads do): every step issues the H2D copies of one batch's keys, offsets
            and features from pinned memory and ends with the D2H copy of one batch's
            probabilities and predictions and a host wait, all inside the timed region
  roofline  the kernel with the largest share of the step, CUDA-event timed in the same run
  cpu_baseline  the CPU oracle (port of the reference's host rule construction and layer
            semantics) on a bounded sample of the same workload, all host cores
  parity    the last timed step of both legs checked, outside the timed regions, against the
            oracle's forward of the same batch: every rulebook equal, largest error of the
            probabilities relative to the largest probability, top-1 agreement; at N > 1 also
            every rank's shard against the oracle's forward of that rank's samples

Every leg is run LEGS times (each --steps long); `value` and `e2e` are the median leg, the
fastest and slowest legs are printed beside them.

--impl reference times that CPU path alone (the reference has no CPU-only executable and
its CUDA kernels are what this library replaces), rank 0 only.
"""
import argparse
import importlib
import json
import os
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG = 2
BATCH_PER_GPU = 256
METRIC = "samples/sec DeepCNet(5,100) fwd"
WORKLOAD = ("config 2: CIFAR-10-shaped dense 32x32x3 N(0,1) patch in a 96x96 grid, DeepCNet(5,100)-style "
            "(conv3 + 5 x conv2, MP2/2, widths 96/192/288/416/512/608 as the reference builder rounds them, "
            "VLeakyReLU, test-time dropout scaling p=0.5 ramp, softmax 10), batch 256 per GPU")


LEGS = 5


def measured_traffic(kernel):
    """DRAM bytes per launch (dram__bytes_read.sum + dram__bytes_write.sum) that a profiler capture of this workload
    recorded for `kernel`: a line "<kernel> <bytes>" of profiles/dram_traffic.txt, None when no capture is on file."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.txt")
    if not os.path.exists(path):
        return None
    for line in open(path):
        f = line.split()
        if len(f) >= 2 and f[0] == kernel:
            return float(f[1])
    return None


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return dict(hbm_gbs=p["hbm_gbs"], tflops=p["bf16_tflops"], tflops_sustained=p.get("bf16_tflops_sustained", p["bf16_tflops"]),
                    source="measured")
    return dict(hbm_gbs=6650.0, tflops=1590.0, tflops_sustained=1400.0, source="fallback")


class ClockSampler:
    """nvidia-smi clocks and throttle reasons of one GPU, sampled every 20 ms."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows, self.proc = [], None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), "--query-gpu=" + self.Q,
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([time.time()] + [x.strip() for x in line.split(",")])

    def wait_first(self, timeout=5.0):
        """Blocks until nvidia-smi has delivered its first sample (its start-up takes a few 100 ms)."""
        t0 = time.time()
        while self.proc is not None and not self.rows and time.time() - t0 < timeout:
            time.sleep(0.01)

    def count_in(self, t0, t1):
        return sum(1 for r in self.rows if t0 <= r[0] <= t1)

    def stop(self, t0=None, t1=None):
        if self.proc is None:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for r in self.rows:
            if (t0 is not None and r[0] < t0) or (t1 is not None and r[0] > t1):
                continue
            r = r[1:]
            try:
                sm.append(float(r[0])); mx.append(float(r[1]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return dict(sm_mhz=float(np.median(sm)) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    reasons=sorted(reasons), samples=len(sm))


def build_pair(scn, want_oracle):
    """The benchmark network in the product and (optionally) in the CPU oracle, same weights."""
    c = scn.synth.CONFIGS[CFG]
    gnet = None
    import torch
    if torch.cuda.is_available():
        gnet = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
        scn.synth.build_network(gnet, CFG)
    onet = None
    if want_oracle:
        from oracle import orc
        onet = orc.OracleNet(orc.Oracle(), c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
        scn.synth.build_network(onet, CFG)
    layers = (gnet or onet).layers()
    for i, (W, B, pr) in scn.synth.init_weights(layers).items():
        if gnet:
            gnet.set_weights(i, W, B, pr)
        if onet:
            onet.set_weights(i, W, B, pr)
    return gnet, onet


def cpu_leg(scn, onet, seconds, threads):
    """Oracle forward over whole batches of the workload until about seconds seconds of wall time."""
    keys, off, feats = scn.synth.CONFIGS[CFG]["gen"](BATCH_PER_GPU)
    keys = keys.astype(np.int64)
    onet.forward(keys[: off[threads]], off[: threads + 1], feats[: off[threads]], threads=threads)  # warm-up
    n, rules_s, t0 = 0, 0.0, time.time()
    while True:
        onet.forward(keys, off, feats, threads=threads)
        n += BATCH_PER_GPU
        rules_s += float(onet.times[0])
        if time.time() - t0 >= seconds:
            break
    wall = time.time() - t0
    return dict(value=n / wall, unit="samples/s", cores=threads, kind="port",
                sample="%d samples (%d batches of %d) of the workload, oracle fp32 forward incl. rule construction, %.1f s wall; "
                       "rule construction alone %.0f samples/s" % (n, n // BATCH_PER_GPU, BATCH_PER_GPU, wall, n / max(rules_s, 1e-9)),
                rules_only_samples_per_s=n / max(rules_s, 1e-9))


def run_reference(args, scn):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    _, onet = build_pair_cpu_only(scn)
    gen = scn.synth.CONFIGS[CFG]["gen"]
    n = BATCH_PER_GPU  # one whole batch per step
    keys, off, feats = gen(n)
    keys = keys.astype(np.int64)
    for _ in range(args.warmup):
        onet.forward(keys[: off[threads]], off[: threads + 1], feats[: off[threads]], threads=threads)
    t0 = time.time()
    rules_s = 0.0
    for _ in range(args.steps):
        onet.forward(keys, off, feats, threads=threads)
        rules_s += float(onet.times[0])
    wall = time.time() - t0
    v = n * args.steps / wall
    line = dict(impl="reference", metric=METRIC, value=v, unit="samples/s", n_gpus=args.gpus, steps=args.steps,
                warmup=args.warmup, ms_per_step=1000.0 * wall / args.steps, higher_is_better=True, scaling="weak",
                vs_baseline=None, dtype="f32", data="synthetic",
                config=dict(workload=WORKLOAD), step="one CPU forward of a bounded sample of %d samples (one batch)" % n,
                cpu_baseline=dict(value=v, unit="samples/s", cores=threads, kind="port",
                                  sample="%d samples per step, %d steps; the reference's host rule construction and "
                                         "layer semantics restated in C++ (oracle), std::thread over samples" % (n, args.steps)),
                e2e=dict(value=v, unit="samples/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line))


def build_pair_cpu_only(scn):
    from oracle import orc
    c = scn.synth.CONFIGS[CFG]
    onet = orc.OracleNet(orc.Oracle(), c["dim"], c["nIn"], c["nClasses"], 1, lattice=c["lattice"])
    scn.synth.build_network(onet, CFG)
    for i, (W, B, pr) in scn.synth.init_weights(onet.layers()).items():
        onet.set_weights(i, W, B, pr)
    return None, onet


def training_side_measurement(scn, n_steps):
    """Outside every timed leg: a few training steps (forward, softmax gradient, every layer's backwards, momentum update;
    host buffers in, probabilities out) of the same layer sequence without dropout, timed by wall clock around the synchronous call."""
    c = scn.synth.CONFIGS[CFG]
    net = scn.net.Net(c["dim"], c["nIn"], c["nClasses"], 1, c["lattice"])
    w, L = c["widths"], len(c["widths"]) - 1
    for i, nf in enumerate(w):
        fs = c.get("first_filter", 3) if i == 0 else 2
        pool = not (c["tail"] == "conv" and i == L)
        net.addLeNetLayerMP(nf, fs, 1, 2 if pool else 1, 2 if pool else 1, scn.synth.VLEAKYRELU, 0.0, 1)
    if c["tail"] == "terminal":
        net.addTerminalPoolingLayer(c["terminal"])
    net.addSoftmaxLayer()
    for i, (W, B, pr) in scn.synth.init_weights(net.layers()).items():
        net.set_weights(i, W, B, pr)
    keys, off, feats = c["gen"](BATCH_PER_GPU)
    labels = (np.arange(BATCH_PER_GPU) % c["nClasses"]).astype(np.int32)
    nll, ms = [], []
    for j in range(n_steps + 1):  # the first step allocates the gradient buffers
        t0 = time.time()
        _, stats = net.train_batch(keys, off, feats, labels, 1e-8, 0.9)  # (a rate small enough for the summed, unnormalised gradients of 256 samples)
        ms.append((time.time() - t0) * 1e3)
        nll.append(stats["nll"] / BATCH_PER_GPU)
    best = min(ms[1:])
    return dict(ms_per_step=best, samples_per_s=BATCH_PER_GPU / (best * 1e-3), steps=n_steps, nll_per_sample=[round(v, 4) for v in nll],
                what="forward + backward + update of the same layers without dropout on one batch repeated, tf32 operands (three products), "
                     "host buffers, wall clock; weight gradients through the fused tensor-core kernel with the roles turned (gathered input transposed, "
                     "gradient packed as the weight operand), input gradients through the same kernel on the transposed weights")


def relerr(a, b):
    return float(np.abs(a - b).max() / max(float(np.abs(b).max()), 1e-30))


def parity_check(scn, gnet, last, world, rank_rows, gathered_host, n_rot, steps, threads):
    """Outside every timed region: the oracle's forward of the batch the last timed step processed, against what both
    legs produced for it.  `last` = dict(batch index, device-leg probabilities and top-1, host-leg probabilities and
    top-1) of this rank.  At N > 1 rank 0 also forwards every other rank's last batch through the oracle and compares
    the all-gathered probabilities and each rank's per-interface row counts with it."""
    _, onet = build_pair_cpu_only(scn)
    gen = scn.synth.CONFIGS[CFG]["gen"]
    j = last["batch_index"]
    keys, off, feats = gen(BATCH_PER_GPU, first=j * BATCH_PER_GPU)
    oprobs, opred = onet.forward(keys.astype(np.int64), off, feats, threads=threads, accum64=True, keep=True)
    layers = gnet.layers()
    rules_equal = True
    for i in range(len(layers) + 1):
        g, o = gnet.iface(i, features=False), onet.iface(i)
        rules_equal = rules_equal and g["nSpatialSites"] == o["nSpatialSites"] and np.array_equal(g["rules"], o["rules"]) \
            and np.array_equal(g["row_keys"], o["row_keys"])
    out = dict(rules_equal=bool(rules_equal),
               max_rel_err=max(relerr(last["dev_probs"], oprobs), relerr(last["host_probs"], oprobs)),
               top1_agree=float(min((last["dev_top"] == opred).mean(), (last["host_top"] == opred).mean())),
               samples=int(len(opred)), checked="last timed step of the device-resident leg and of the host-buffer leg vs the oracle "
               "(fp64 accumulation); rulebooks and grids of every interface")
    if world > 1:
        ok, worst = True, 0.0
        for r in range(world):
            k2, o2, f2 = gen(BATCH_PER_GPU, first=(r * n_rot + (steps - 1) % n_rot) * BATCH_PER_GPU)
            p2, _ = onet.forward(k2.astype(np.int64), o2, f2, threads=threads, accum64=True, keep=True)
            rows = [onet.iface(i)["nSpatialSites"] for i in range(len(layers) + 1)]
            ok = ok and rows == [int(v) for v in rank_rows[r]]
            worst = max(worst, relerr(gathered_host[r * BATCH_PER_GPU:(r + 1) * BATCH_PER_GPU], p2))
        out["shards_equal_whole"] = bool(ok and worst < 1e-4)
        out["shards_max_rel_err"] = worst
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--precision", default="auto", choices=["auto", "split", "fp32", "3xtf32", "bf16", "3xbf16"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0, help="wall time of the cpu_baseline leg (0 = skip it and the parity check)")
    ap.add_argument("--config", type=int, default=2, choices=[1, 2, 3, 4, 5],
                    help="synthetic configuration (2 = the headline workload; the others are side measurements)")
    ap.add_argument("--batch", type=int, default=0, help="samples per GPU (0 = the configuration's own batch size, at most 256)")
    ap.add_argument("--train-steps", type=int, default=3, help="training steps of the side measurement (0 = skip it)")
    ap.add_argument("--legs", type=int, default=LEGS, help="how often each timed leg is repeated (the median leg is reported)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "native" else args.warmup

    scn = importlib.import_module("sparseconvnet-archived_b200")
    global CFG, BATCH_PER_GPU, WORKLOAD
    if args.config != 2 or args.batch:
        CFG = args.config
        BATCH_PER_GPU = args.batch or min(256, scn.synth.CONFIGS[CFG]["batch"])
        if CFG != 2:
            WORKLOAD = "config %d of the benchmark description (side measurement), batch %d per GPU" % (CFG, BATCH_PER_GPU)
    if args.impl == "reference":
        run_reference(args, scn)
        return

    import torch
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert torch.cuda.is_available(), "bench.py needs a CUDA device (there is no CPU fallback)"
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    dev = torch.device("cuda", local)
    abi = scn.abi
    stream = torch.cuda.Stream(device=dev)
    c = scn.synth.CONFIGS[CFG]
    nC = c["nClasses"]
    peaks = measured_peaks()
    steps = args.steps

    with torch.cuda.stream(stream):
        gnet, _ = build_pair(scn, False)
        gnet.set_precision(dict(auto=abi.PREC_AUTO, split=abi.PREC_SPLIT, fp32=abi.PREC_FP32, **{"3xtf32": abi.PREC_3XTF32, "3xbf16": abi.PREC_3XBF16}, bf16=abi.PREC_BF16)[args.precision])
        # this rank's shard of the global batch, several distinct batches rotated between steps
        n_rot = 2
        host_batches = [c["gen"](BATCH_PER_GPU, first=(rank * n_rot + j) * BATCH_PER_GPU) for j in range(n_rot)]
        # the host-buffer leg reads its inputs from pinned (page-locked) host memory
        pinned_keep = [[torch.from_numpy(np.ascontiguousarray(x)).pin_memory() for x in hb] for hb in host_batches]
        host_batches = [tuple(t.numpy() for t in hb) for hb in pinned_keep]
        dev_batches = []
        for keys, off, feats in host_batches:
            bg = off[:-1].copy()  # the background row is each sample's first row
            dev_batches.append(tuple(torch.from_numpy(x).to(dev) for x in (keys, off, bg, feats)) + (int(np.diff(off).max() - 1),))
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
        d_top = torch.empty((BATCH_PER_GPU, 1), dtype=torch.int32, device=dev)
        # At N > 1 every rank's probabilities go to every rank over peer memory (ResultExchange: the forward call stores
        # its block into the peers' buffers and collects the step before in front of its one copy-and-wait; no collective
        # call per step).  The blocks of step j are therefore delivered by step j + 1, in both legs; the last step's
        # blocks are collected, and timed, behind the last step.
        d_probs2 = [torch.empty((BATCH_PER_GPU, nC), dtype=torch.float32, device=dev) for _ in range(2)]
        gathered2 = [torch.zeros((world * BATCH_PER_GPU, nC), dtype=torch.float32, device=dev) for _ in range(2)]
        d_rows_status = torch.zeros(world + 1, dtype=torch.int32, device=dev)
        h_gathered = np.zeros((world, BATCH_PER_GPU, nC), np.float32)
        h_rows = np.zeros(world, np.int32)
        pending = []
        last_host = {}
        # (should the buffers not map on this machine, every rank falls back to an NCCL all-gather per step, gather of
        # step j on NCCL's stream while step j + 1 computes: the line's config says which one ran)
        exchange = world > 1 and os.environ.get("SCN_EXCHANGE", "1") != "0" and scn.shard.connect_exchange(gnet, BATCH_PER_GPU)
        h_gathered_pinned = torch.empty((world * BATCH_PER_GPU, nC), dtype=torch.float32).pin_memory() if world > 1 and not exchange else None

        def step_device(j):
            dk, do, db, df, ms = dev_batches[j % n_rot]
            gnet.forward_device(dk, do, db, df, ms, d_probs2[j & 1], d_top)
            if world == 1:
                return
            if exchange:  # collects step j - 1 into gathered2[(j - 1) & 1], publishes step j
                gnet.exchange_step_device(d_probs2[j & 1], BATCH_PER_GPU, gathered2[(j - 1) & 1], d_rows_status)
                pending[:] = [("device", j & 1)]
            else:
                work = dist.all_gather_into_tensor(gathered2[j & 1], d_probs2[j & 1], async_op=True)
                drain()  # the launching stream waits for the previous step's gather
                pending.append(("nccl", work, j & 1, False))

        def drain():
            while pending:
                entry = pending.pop()
                if entry[0] == "device":
                    gnet.exchange_step_device(None, 0, gathered2[entry[1]], d_rows_status)
                elif entry[0] == "host":  # the host leg's last step: its blocks come back to the host
                    gnet.exchange_flush(h_gathered, h_rows)
                else:
                    _, work, k, to_host = entry
                    work.wait()
                    if to_host:
                        h_gathered_pinned.copy_(gathered2[k], non_blocking=True)
                        stream.synchronize()

        run = {"n": steps}  # length of the run of steps under way (the host leg begins batch j + 1 before it ends batch j)

        def step_host(j):
            # forward_host in two halves: the inputs of batch j + 1 start their way to the device, then batch j (begun by
            # the previous step) is computed and its results are waited for.  Every step issues one batch's copies and
            # returns one batch's results; the first step of a run issues two batches' copies, the last one none.
            if j == 0:
                gnet.forward_host_begin(*host_batches[0])
            if j + 1 < run["n"]:
                gnet.forward_host_begin(*host_batches[(j + 1) % n_rot])
            if world == 1 or not exchange:
                probs, pred = gnet.forward_host_end()
            else:
                probs, pred, _, _ = gnet.forward_host_end(True, h_gathered, h_rows)
                pending[:] = [("host", 0)]
            last_host["probs"], last_host["top"] = probs, pred
            if world > 1 and not exchange:
                gnet.copy_probs_device(d_probs2[j & 1])
                work = dist.all_gather_into_tensor(gathered2[j & 1], d_probs2[j & 1], async_op=True)
                drain()
                pending.append(("nccl", work, j & 1, True))

        def timed(step, with_layer_times):
            ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
            layer_ms = None
            for j in range(steps):
                flush.fill_(j & 0xff)
                ev[j][0].record(stream)
                step(j)
                ev[j][1].record(stream)
                if with_layer_times:
                    t = gnet.layer_times()  # waits for the stream
                    layer_ms = t if layer_ms is None else layer_ms + t
            tail = None
            if pending:  # the last step's gather: timed after its step
                tail = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                tail[0].record(stream)
                drain()
                tail[1].record(stream)
            stream.synchronize()
            ms = sum(a.elapsed_time(b) for a, b in ev)
            if tail:
                ms += tail[0].elapsed_time(tail[1])
            return ms, (layer_ms / steps if layer_ms is not None else None)

        def barrier():
            stream.synchronize()
            if world > 1:
                dist.barrier()
            torch.cuda.synchronize()

        def check_tc(leg):
            code = abi.conv_tc_take_error()
            if code:
                raise RuntimeError("a tensor-core kernel gave up a time-limited wait (code %d) during the %s leg: its numbers are void" % (code, leg))

        def legs(step):
            out = []
            for _ in range(max(1, args.legs)):
                barrier()
                ms, _ = timed(step, False)
                barrier()
                out.append(ms)
            return out

        # ---- device-resident leg
        sampler = ClockSampler(local)
        sampler.wait_first()
        for j in range(args.warmup):
            step_device(j)
        drain()
        barrier()
        t_load0 = time.time()
        launches0 = abi.kernel_launch_count()
        t_wall = time.time()
        ms_dev_legs = legs(step_device)
        t_wall = time.time() - t_wall
        launches = (abi.kernel_launch_count() - launches0) // max(1, args.legs)
        check_tc("device-resident")
        last = dict(batch_index=rank * n_rot + (steps - 1) % n_rot, dev_probs=d_probs2[(steps - 1) & 1].cpu().numpy(), dev_top=d_top.cpu().numpy())
        gathered_host = gathered2[(steps - 1) & 1].cpu().numpy() if world > 1 else None
        if world > 1 and exchange and int(d_rows_status[world].item()):
            raise RuntimeError("the result exchange gave up waiting for ranks (bits %d): this leg's numbers are void" % int(d_rows_status[world].item()))
        # Per-kernel durations for the roofline and the breakdown: the same steps once more with a CUDA
        # event between the layers.  (Those events cost about 0.06 ms of GPU idle per step, which is why
        # they are kept out of the steps that `value` is computed from.)
        gnet.enable_timing(True)
        _, layer_ms = timed(step_device, True)
        barrier()
        gnet.enable_timing(False)
        # ---- host-buffer leg
        run["n"] = args.warmup
        for j in range(args.warmup):
            step_host(j)
        drain()
        run["n"] = steps
        ms_e2e_legs = legs(step_host)
        check_tc("host-buffer")
        last["host_probs"], last["host_top"] = last_host["probs"].copy(), last_host["top"].copy()
        # A short run (few steps) can end between two nvidia-smi samples: keep the same steps going,
        # untimed, until a handful of samples have been taken under this load.
        tail_ms, j = 0.0, 0
        t_tail = time.time()
        # (no collective in here: every rank runs its own number of extra steps)
        while sampler.proc is not None and sampler.count_in(t_load0, time.time()) < 5 and time.time() - t_tail < 2.0:
            dk, do, db, df, ms = dev_batches[j % n_rot]
            gnet.forward_device(dk, do, db, df, ms, d_probs2[0], d_top)
            j += 1
        if j:
            stream.synchronize()
            tail_ms = (time.time() - t_tail) * 1e3
        clocks = sampler.stop(t_load0, time.time())
        clocks["window"] = "all timed legs" + (" + %.0f ms of the same steps, untimed" % tail_ms if j else "")
        # leave the network holding the last timed batch of the host leg (the parity check reads its rulebooks)
        gnet.forward_host(*host_batches[(steps - 1) % n_rot])

        # shapes of the last forward for the roofline arithmetic
        layers = gnet.layers()
        sizes = [gnet.iface(i, features=False) for i in range(len(layers) + 1)]

    # every leg: max over ranks, then the median leg
    t = torch.tensor([ms_dev_legs, ms_e2e_legs], dtype=torch.float64, device=dev)
    rows_t = torch.tensor([sz["nSpatialSites"] for sz in sizes], dtype=torch.int64, device=dev)
    rank_rows = [rows_t.cpu().numpy()]
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        allrows = torch.empty((world, rows_t.numel()), dtype=torch.int64, device=dev)
        dist.all_gather_into_tensor(allrows, rows_t)
        rank_rows = allrows.cpu().numpy()
    dev_legs, e2e_legs = (sorted(float(x) for x in row) for row in t.cpu())
    ms_dev, ms_e2e = dev_legs[len(dev_legs) // 2], e2e_legs[len(e2e_legs) // 2]
    total = world * BATCH_PER_GPU * steps

    # ---- roofline of the kernel with the largest share of the step
    per_layer = []
    for i, L in enumerate(layers):
        rows_in, rows_out = sizes[i]["nSpatialSites"], sizes[i + 1]["nSpatialSites"]
        ms = float(layer_ms[i])
        if L["type"] == 2:
            fused = i > 0 and layers[i - 1]["type"] in (0, 1)
            fs = layers[i - 1]["fs"] if fused else 1
            src_rows = sizes[i - 1]["nSpatialSites"] if fused else rows_in
            K, N = L["nIn"], L["nOut"]
            flops = 2.0 * rows_out * K * N
            byts = 4.0 * (src_rows * (K // fs) + (rows_out * fs if fused else 0) + K * N + N + rows_out * N)
            per_layer.append(dict(layer=i, kernel="conv_nin_fused" if fused else "nin", rows=rows_out, K=K, N=N, ms=ms,
                                  flops=flops, bytes=byts))
        elif L["type"] in (3, 4):
            C = sizes[i + 1]["nFeatures"]
            byts = 4.0 * (rows_out * L["fs"] + rows_in * C + 2 * rows_out * C)
            per_layer.append(dict(layer=i, kernel="maxpool_rules", rows=rows_out, C=C, ms=ms, flops=0.0, bytes=byts))
    # A learnt layer that a non-overlapping max pooling follows leaves its output to the pooling layer; where that
    # layer ran convolution, learnt layer and pooling as one kernel (layer info `act` = 1) the two are one launch.
    merged = []
    for d in per_layer:
        prev = merged[-1] if merged else None
        if (d["kernel"] == "maxpool_rules" and layers[d["layer"]]["act"] == 1 and prev is not None
                and prev["kernel"] == "conv_nin_fused" and prev["layer"] == d["layer"] - 1):
            prev["kernel"] = "conv_nin_maxpool_fused"
            prev["ms"] += d["ms"]
            prev["bytes"] += 4.0 * (d["rows"] * layers[d["layer"]]["fs"] + 2 * d["rows"] * d["C"] - prev["rows"] * prev["N"])
            prev["pooled_rows"] = d["rows"]
        else:
            merged.append(d)
    per_layer = merged
    rules_ms = float(layer_ms[len(layers)])
    # The dominant kernel of the step is the tensor-core fused conv/NiN kernel (k_conv_nin_tc): its
    # launches with K >= 128 are tensor-bound, so the roofline entry is their algorithmic flops per
    # launch over their average launch time, against the measured bf16 figure of a kernel timed alone
    # (these launches last 25-70 us).  kind::tf32 runs at half the bf16 rate and 3xTF32 issues three MMAs
    # per product: `pipe_frac` is the same time against that ceiling (peak / 6).
    tc = [d for d in per_layer if d["kernel"] != "maxpool_rules" and d.get("K", 0) >= 128 and d["N"] >= 16]
    step_ms = ms_dev / steps
    # tensor-pipe passes per product against the bf16 rate: three bf16 products for the layers with K >= 128 (auto / split),
    # three tf32 products at half the bf16 rate for 3xtf32
    passes = {"auto": 3.0, "split": 3.0, "3xtf32": 6.0, "3xbf16": 3.0, "bf16": 1.0}.get(args.precision, 3.0)
    if tc and args.precision != "fp32":
        ach = sum(d["flops"] for d in tc) / (sum(d["ms"] for d in tc) * 1e-3) / 1e12
        roof = dict(bound="tensor", achieved=ach, peak=peaks["tflops"], unit="TFLOP/s", frac=ach / peaks["tflops"],
                    traffic=measured_traffic("k_conv_nin_tc") if (world == 1 and CFG == 2 and BATCH_PER_GPU == 256) else None,
                    kernel="k_conv_nin_tc (%d launches per step with K >= 128, %d of them with the max pooling fused in)" % (len(tc), sum(d["kernel"] == "conv_nin_maxpool_fused" for d in tc)),
                    ms_per_launch=sum(d["ms"] for d in tc) / len(tc), share_of_step=sum(d["ms"] for d in tc) / step_ms,
                    frac_of_sustained_peak=ach / peaks["tflops_sustained"], pipe_frac=ach * passes / peaks["tflops"],
                    note="peak is the measured bf16 cuBLAS burst figure; these layers (K >= 128) run the three-product split on bf16 operands "
                         "(auto / split; three tf32 products at half the rate for 3xtf32), so 1/3 (1/6) of this peak is the ceiling of a perfect "
                         "kernel: pipe_frac is against that ceiling")
    else:
        top = max(per_layer, key=lambda d: d["ms"])
        ach = top["bytes"] / (top["ms"] * 1e-3) / 1e9
        roof = dict(bound="hbm", achieved=ach, peak=peaks["hbm_gbs"], unit="GB/s", frac=ach / peaks["hbm_gbs"], traffic=None,
                    kernel="layer %d %s" % (top["layer"], top["kernel"]), ms_per_launch=top["ms"], share_of_step=top["ms"] / step_ms)
    roof["peak_source"] = peaks["source"]
    # the HBM side: pooling as a kernel of its own, and the fused convolution + pooling kernels against the same 70 % bar
    hbm_side = []
    for d in per_layer:
        if d["kernel"] in ("maxpool_rules", "conv_nin_maxpool_fused") or d.get("K", 1 << 30) < 128:
            gbs = d["bytes"] / (d["ms"] * 1e-3) / 1e9
            hbm_side.append(dict(layer=d["layer"], kernel=d["kernel"], gbs=gbs, frac=gbs / peaks["hbm_gbs"]))
    pool = [d for d in per_layer if d["kernel"] == "maxpool_rules"]
    pool_top = max(pool, key=lambda d: d["ms"]) if pool else None
    all_flops = sum(d["flops"] for d in per_layer)
    conv_ms = sum(d["ms"] for d in per_layer if d["kernel"] != "maxpool_rules")

    training = None
    if rank == 0 and args.train_steps > 0:
        try:
            with torch.cuda.stream(stream):
                training = training_side_measurement(scn, args.train_steps)
        except Exception as e:  # a side measurement must not take the benchmark line with it
            training = dict(unavailable=str(e))
    if rank == 0:
        cpu, parity = None, None
        if args.cpu_seconds > 0:
            try:
                _, onet = build_pair_cpu_only(scn)
                cpu = cpu_leg(scn, onet, args.cpu_seconds, os.cpu_count() or 1)
                parity = parity_check(scn, gnet, last, world, rank_rows, gathered_host, n_rot, steps, os.cpu_count() or 1)
            except Exception as e:  # the oracle is a checker, its absence must not hide the GPU numbers
                cpu = cpu or dict(value=None, unit="samples/s", cores=0, kind="port", sample="unavailable: %s" % e)
                parity = parity or dict(unavailable=str(e))
        h2d = int(sum(x.nbytes for x in host_batches[0]))
        d2h = int(BATCH_PER_GPU * nC * 4 + BATCH_PER_GPU * 4 + 4 + (world * BATCH_PER_GPU * nC * 4 + (world + 1) * 4 if world > 1 else 0))
        line = dict(
            metric=METRIC, value=total / (ms_dev * 1e-3), unit="samples/s", n_gpus=world, steps=steps, warmup=args.warmup,
            ms_per_step=ms_dev / steps, higher_is_better=True, scaling="weak", vs_baseline=None,
            dtype={"fp32": "f32", "bf16": "bf16", "3xtf32": "tf32x3/f32", "3xbf16": "bf16x3/f32"}.get(args.precision, "bf16x3|tf32x3/f32"), data="synthetic",
            config=dict(workload=WORKLOAD, global_batch=world * BATCH_PER_GPU, parallelism="dp%d by sample%s" % (world, "" if world == 1 else ", every rank's probabilities stored into every rank's buffer over peer memory by the forward call (no collective call per step); step j's blocks are delivered by step j+1 in both legs, the last step's behind it" if exchange else ", NCCL all-gather of the probabilities per step (the peer-memory exchange could not be set up here), overlapped with the next step"),
                        l2="256 MiB written between timed steps; 2 distinct batches rotated", precision=args.precision,
                        timing="CUDA events per step on the launching stream, max over ranks; each leg %d times, median leg reported; wall %.3f s for the device legs; per-kernel durations from one more pass of the same steps with events between the layers" % (max(1, args.legs), t_wall)),
            legs=dict(n=max(1, args.legs), ms_per_step_device=[round(x / steps, 5) for x in dev_legs], ms_per_step_e2e=[round(x / steps, 5) for x in e2e_legs]),
            e2e=dict(value=total / (ms_e2e * 1e-3), unit="samples/s", h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h,
                     call="scn_net_forward_host_begin / _end: each step starts the copies of the next batch, then computes and returns the current one",
                     ms_per_step=ms_e2e / steps),
            gpu_launches=int(launches), roofline=roof, cpu_baseline=cpu, parity=parity, clocks=clocks, training_step=training,
            pooling_roofline=(dict(bound="hbm", kernel="k_maxpool layer %d" % pool_top["layer"], achieved=pool_top["bytes"] / (pool_top["ms"] * 1e-3) / 1e9,
                                   peak=peaks["hbm_gbs"], unit="GB/s", frac=pool_top["bytes"] / (pool_top["ms"] * 1e-3) / 1e9 / peaks["hbm_gbs"])
                              if pool_top else None),
            hbm_side=hbm_side,
            breakdown=dict(rule_chain_ms=rules_ms, conv_nin_ms=conv_ms, conv_algorithmic_tflops=all_flops / (conv_ms * 1e-3) / 1e12,
                           multiply_adds_per_sample=all_flops / 2 / BATCH_PER_GPU,
                           layers=[dict(layer=d["layer"], kernel=d["kernel"], ms=round(d["ms"], 4), rows=d["rows"],
                                        gflop=round(d["flops"] / 1e9, 3), mbytes=round(d["bytes"] / 1e6, 2),
                                        **({"pipe_frac": round(d["flops"] / (d["ms"] * 1e-3) / 1e12 * passes / peaks["tflops"], 3)} if d.get("K", 0) >= 128 and d.get("N", 0) >= 16 else {}))
                                   for d in per_layer]),
        )
        print(json.dumps(line))
    if world > 1:
        if exchange:
            scn.shard.disconnect_exchange(gnet)
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
