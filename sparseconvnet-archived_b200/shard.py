"""Sharding of a batch over ranks: samples are independent through every layer (rules, gather
and pooling are per sample, the GEMM is row-wise), so rank r simply takes a contiguous block
of samples, builds its own rulebooks and runs its own forward; the single exchange step is an
all-gather of the final class probabilities.  On the GPUs of one node that step runs over peer
memory inside the forward call (connect_exchange, then Net.forward_host_exchange /
Net.exchange_step_device: no collective call per step); gather_probabilities / gather_ragged do
the same through torch.distributed for any backend (NCCL on GPUs, gloo in the CPU tests)."""
import numpy as np
import torch
import torch.distributed as dist


def shard_range(n_samples, rank, world):
    """Contiguous block [lo, hi) of samples for `rank`, sizes differing by at most one."""
    base, extra = divmod(n_samples, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def balanced_ranges(site_counts, world):
    """Contiguous blocks with nearly equal numbers of ACTIVE SITES (the cost driver when samples
    differ in size).  Returns world+1 boundaries."""
    c = np.concatenate([[0], np.cumsum(np.asarray(site_counts, np.int64))])
    total = c[-1]
    bounds = [0]
    for r in range(1, world):
        target = total * r / world
        i = int(np.searchsorted(c, target, side="left"))
        i = min(max(i, bounds[-1]), len(site_counts))
        # pick the nearer of the two candidate cuts
        if i > bounds[-1] and abs(c[i - 1] - target) <= abs(c[i] - target):
            i -= 1
        bounds.append(max(i, bounds[-1]))
    bounds.append(len(site_counts))
    return bounds


def take_samples(keys, off, feats, lo, hi):
    """Slice a flat batch (keys, off, feats) to samples [lo, hi), renumbering rows from 0."""
    r0, r1 = int(off[lo]), int(off[hi])
    return keys[r0:r1], (off[lo:hi + 1] - r0).astype(np.int32), feats[r0:r1]


def gather_probabilities(local, group=None):
    """All-gather equal-sized [n x C] blocks into [world*n x C] in rank order."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    out = torch.empty((dist.get_world_size(group) * local.shape[0],) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(out, local.contiguous(), group=group)
    return out


def gather_ragged(local, counts, group=None):
    """All-gather [n_r x C] blocks of different sizes (counts[r] rows from rank r): pad to the
    largest, gather, cut."""
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return local
    m = int(max(counts))
    pad = torch.zeros((m,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[: local.shape[0]] = local
    g = gather_probabilities(pad, group)
    return torch.cat([g[r * m: r * m + int(counts[r])] for r in range(len(counts))])


def _all_ok(ok, dev, group):
    flag = torch.tensor([1 if ok else 0], dtype=torch.int32, device=dev)
    dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
    return bool(int(flag.item()))


def connect_exchange(net, cap_rows, group=None):
    """Sets up the peer-memory result exchange of `net` among the ranks of `group` (one process per GPU, one node):
    every rank allocates its buffer, the 64-byte handles travel once through torch.distributed, every rank maps the
    others' buffers.  cap_rows = the largest number of samples a rank will publish in one step.  Returns True when
    EVERY rank succeeded; otherwise every rank has dropped its half-built exchange and gets False (the caller falls
    back to gather_probabilities).  Ranks agree after each local step, so no rank is left alone in a collective."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    dev = torch.device("cuda", torch.cuda.current_device()) if dist.get_backend(group) == "nccl" else torch.device("cpu")
    handle, ok = bytes(64), True
    try:
        handle = net.exchange_create(world, rank, cap_rows)
    except Exception:
        ok = False
    if not _all_ok(ok, dev, group):
        net.exchange_destroy()
        return False
    mine = torch.tensor(list(handle), dtype=torch.uint8, device=dev)
    everyone = [torch.empty_like(mine) for _ in range(world)]
    dist.all_gather(everyone, mine, group=group)
    try:
        net.exchange_connect(b"".join(bytes(t.cpu().tolist()) for t in everyone))
    except Exception:
        ok = False
    if not _all_ok(ok, dev, group):  # (also the point behind which everybody has mapped everybody: publishing may start)
        torch.cuda.synchronize()
        dist.barrier(group)
        net.exchange_destroy()
        return False
    return True


def disconnect_exchange(net, group=None):
    """Every rank has stopped publishing (its stream is idle) before any rank frees its buffer."""
    torch.cuda.synchronize()
    dist.barrier(group)
    net.exchange_destroy()
    dist.barrier(group)
