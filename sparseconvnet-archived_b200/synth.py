"""Seeded synthetic workloads with the shapes, sizes and value distributions of the five
benchmark configurations, and weight initialisation.  They stand in for the datasets the
reference's loaders expect (image, pen-stroke, 3-D shape and video sets), none of which ships
with it.  Sample s of configuration c is drawn from numpy's default_rng(1000*c + s).

Each generator returns a batch in the flat input form of scn_net_forward_host:
    keys  int32 [rows]  site key per row (row-major index in the S^dim cube), -1 for the
                        sample's background row, which comes first as the reference's
                        Picture classes emit it
    off   int32 [batch+1]
    feats float32 [rows x nInputFeatures]  (background rows are zero)
"""
import numpy as np

from . import abi

VLEAKYRELU = abi.VLEAKYRELU


def _assemble(samples, nF):
    keys, feats, off = [], [], [0]
    for k, f in samples:
        keys.append(np.concatenate([[-1], k]).astype(np.int32))
        feats.append(np.concatenate([np.zeros((1, nF), np.float32), f.astype(np.float32)]))
        off.append(off[-1] + len(k) + 1)
    return np.concatenate(keys), np.array(off, np.int32), np.concatenate(feats)


def _unique_keep_order(k):
    _, idx = np.unique(k, return_index=True)
    return k[np.sort(idx)]


def config1(batch, first=0):
    """2-D pen strokes: 3 random walks of 40 unit steps (8 directions) on a 48x48 grid,
    3 features uniform[-1,1] per site."""
    S, out = 48, []
    dirs = np.array([(dx, dy) for dx in (-1, 0, 1) for dy in (-1, 0, 1) if dx or dy])
    for s in range(first, first + batch):
        rng = np.random.default_rng(1000 * 1 + s)
        pts = []
        for _ in range(3):
            p = rng.integers(0, S, 2)
            pts.append(p.copy())
            for d in dirs[rng.integers(0, 8, 40)]:
                p = np.clip(p + d, 0, S - 1)
                pts.append(p.copy())
        pts = np.array(pts)
        k = _unique_keep_order(pts[:, 0] * S + pts[:, 1])
        out.append((k, rng.uniform(-1, 1, (len(k), 3))))
    return _assemble(out, 3)


def config2(batch, first=0):
    """CIFAR-10-shaped: a dense 32x32 patch of 3 N(0,1) channels centred in a 96x96 grid."""
    S, out = 96, []
    x, y = np.meshgrid(np.arange(32, 64), np.arange(32, 64), indexing="ij")
    k = (x * S + y).ravel()
    for s in range(first, first + batch):
        rng = np.random.default_rng(1000 * 2 + s)
        out.append((k, rng.standard_normal((len(k), 3))))
    return _assemble(out, 3)


def _surface_points(rng, S):
    """Points on a randomly rotated ellipsoid or torus (radii 8-20 voxels) whose surface is
    displaced along its normal by a smooth Gaussian field of standard deviation 1 voxel,
    centred in an S^3 box."""
    n = 80000
    if rng.random() < 0.5:
        r = rng.uniform(8, 20, 3)
        v = rng.standard_normal((n, 3))
        v /= np.linalg.norm(v, axis=1, keepdims=True)
        p, nrm = v * r, v
    else:
        R, r = rng.uniform(12, 20), rng.uniform(8, 12) / 2
        u, w = rng.uniform(0, 2 * np.pi, n), rng.uniform(0, 2 * np.pi, n)
        nrm = np.stack([np.cos(w) * np.cos(u), np.cos(w) * np.sin(u), np.sin(w)], 1)
        p = np.stack([R * np.cos(u), R * np.sin(u), np.zeros(n)], 1) + r * nrm
    M = 8  # random plane waves: a smooth field with unit variance
    wv = rng.standard_normal((M, 3)) * 0.25
    ph = rng.uniform(0, 2 * np.pi, M)
    amp = rng.standard_normal(M) * np.sqrt(2.0 / M)
    g = (np.sin(p @ wv.T + ph) * amp).sum(1)
    p = p + nrm * g[:, None]
    q, _ = np.linalg.qr(rng.standard_normal((3, 3)))
    return p @ q.T + S / 2.0


def config3(batch, first=0, S=48):
    """3-D surface voxels of a random ellipsoid or torus in a 48^3 grid, 1 feature = 1.0."""
    out = []
    for s in range(first, first + batch):
        rng = np.random.default_rng(1000 * 3 + s)
        v = np.floor(_surface_points(rng, S)).astype(np.int64)
        v = v[((v >= 0) & (v < S)).all(1)]
        k = _unique_keep_order(v[:, 0] * S * S + v[:, 1] * S + v[:, 2])
        out.append((k, np.ones((len(k), 1))))
    return _assemble(out, 1)


def config4(batch, first=0, S=47):
    """The same shapes rasterised on a tetrahedral lattice of side S: coordinates are mapped by
    the tetrahedron-to-simplex matrix and kept iff all are >= 0 and sum < S."""
    out = []
    M = np.array([[1, -1 / np.sqrt(3), -1 / np.sqrt(6)], [0, 2 / np.sqrt(3), -1 / np.sqrt(6)], [0, 0, np.sqrt(1.5)]])
    for s in range(first, first + batch):
        rng = np.random.default_rng(1000 * 4 + s)
        p = (_surface_points(rng, 0) * 0.45) @ M.T + S / 4.0
        v = np.floor(p).astype(np.int64)
        v = v[(v >= 0).all(1) & (v.sum(1) < S)]
        k = _unique_keep_order(v[:, 0] * S * S + v[:, 1] * S + v[:, 2])
        out.append((k, np.ones((len(k), 1))))
    return _assemble(out, 1)


def config5(batch, first=0, S=64, density=0.05):
    """Space-time volume 64x64x32 (t in [16,48) of a cubic 64^3 grid): 20 moving Gaussian
    blobs activating about 5% of the 131072 cells, 3 N(0,1) features per site."""
    out = []
    for s in range(first, first + batch):
        rng = np.random.default_rng(1000 * 5 + s)
        field = np.zeros((S, S, 32), np.float32)
        t = np.arange(32)
        xx, yy = np.meshgrid(np.arange(S), np.arange(S), indexing="ij")
        for _ in range(20):
            p0, vel, sig = rng.uniform(8, S - 8, 2), rng.uniform(-1, 1, 2), rng.uniform(1.0, 2.5)
            cx, cy = p0[0] + vel[0] * t, p0[1] + vel[1] * t
            field += np.exp(-((xx[..., None] - cx) ** 2 + (yy[..., None] - cy) ** 2) / (2 * sig * sig))
        field += 0.02 * rng.random(field.shape).astype(np.float32)
        thr = np.quantile(field, 1 - density)
        x, y, tt = np.nonzero(field > thr)
        k = x.astype(np.int64) * S * S + y * S + (tt + 16)
        out.append((k, rng.standard_normal((len(k), 3))))
    return _assemble(out, 3)


CONFIGS = {
    1: dict(dim=2, nIn=3, nClasses=10, grid=48, widths=(32, 64, 96, 128, 160), gen=config1, batch=32, lattice=0, tail="conv"),
    2: dict(dim=2, nIn=3, nClasses=10, grid=96, widths=(100, 200, 300, 400, 500, 600), gen=config2, batch=256, lattice=0, tail="conv", p=0.5),
    3: dict(dim=3, nIn=1, nClasses=20, grid=48, widths=(32, 64, 96, 128, 160), gen=config3, batch=64, lattice=0, tail="conv"),
    4: dict(dim=3, nIn=1, nClasses=20, grid=47, widths=(32, 64, 96, 128), gen=config4, batch=64, lattice=1, tail="terminal", first_filter=2, terminal=2),
    5: dict(dim=3, nIn=3, nClasses=101, grid=64, widths=(64, 128, 192, 256), gen=config5, batch=512, lattice=0, tail="terminal", terminal=3),
}


def build_network(net, cfg):
    """Issue the builder calls of configuration `cfg` on `net`, any object with the facade's
    addLeNetLayerMP / addTerminalPoolingLayer(poolSize) / addSoftmaxLayer methods.
    "addLeNetLayerMP-style DeepCNet": conv (3 first, then 2) + MP2/2 per level; the last level
    has no pooling ("conv" tail) or every level pools and terminal pooling follows."""
    c = CONFIGS[cfg]
    w = c["widths"]
    p = c.get("p", 0.0)
    L = len(w) - 1
    for i, nf in enumerate(w):
        fs = c.get("first_filter", 3) if i == 0 else 2
        pool = not (c["tail"] == "conv" and i == L)
        dropout = p * i / L if L else 0.0
        net.addLeNetLayerMP(nf, fs, 1, 2 if pool else 1, 2 if pool else 1, VLEAKYRELU, dropout, 1)
    if c["tail"] == "terminal":
        net.addTerminalPoolingLayer(c["terminal"])
    net.addSoftmaxLayer()


def init_weights(layers, seed=7):
    """He-normal weights (variance 2/K) and N(0, 0.01^2) biases for every learnt layer of a
    layer list (as returned by Net.layers() / OracleNet.layers()): {layer index: (W, B, prelu)}."""
    out = {}
    for i, L in enumerate(layers):
        if L["type"] != 2:
            continue
        rng = np.random.default_rng(seed + i)
        K, N = L["nIn"], L["nOut"]
        W = (rng.standard_normal((K, N)) * np.sqrt(2.0 / K)).astype(np.float32)
        B = (rng.standard_normal(N) * 0.01).astype(np.float32)
        out[i] = (W, B, None)
    return out
