"""Generates tests/golden/rules_golden.npz from the REFERENCE's own rule builder
(oracle/_ref/libscn_ref.so, i.e. Regions.cu compiled unchanged).  Run where the reference
checkout is mounted:  python tests/golden/make_golden.py
The fixtures let the oracle and the GPU path be checked on machines without the reference."""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, os.path.dirname(HERE))
from gridgen import random_grids  # noqa: E402
from oracle import orc  # noqa: E402

# name: (lattice, dim, nOut, size, stride, minActive, batch, density)
CASES = {
    "sq2_conv3": (0, 2, 6, 3, 1, 1, 3, 0.2),
    "sq2_pool2": (0, 2, 5, 2, 2, 1, 3, 0.3),
    "sq2_pool3s2": (0, 2, 4, 3, 2, 1, 2, 0.5),
    "sq3_conv3": (0, 3, 4, 3, 1, 1, 2, 0.1),
    "sq3_conv2": (0, 3, 5, 2, 1, 1, 2, 0.3),
    "sq3_pool2": (0, 3, 3, 2, 2, 1, 2, 0.4),
    "sq2_min2": (0, 2, 6, 3, 1, 2, 3, 0.15),
    "sq3_min3": (0, 3, 4, 2, 1, 3, 2, 0.4),
    "sq2_valid": (0, 2, 7, 3, 1, -1, 2, 0.5),
    "sq1_conv3": (0, 1, 9, 3, 1, 1, 2, 0.4),
    "tri2_conv2": (1, 2, 6, 2, 1, 1, 3, 0.3),
    "tri3_conv2": (1, 3, 5, 2, 1, 1, 2, 0.3),
    "tri3_pool2": (1, 3, 4, 2, 2, 1, 2, 0.4),
    "tri3_min2": (1, 3, 5, 2, 1, 2, 2, 0.3),
    "tri2_min3": (1, 2, 5, 3, 1, 3, 2, 0.5),
    "sq2_full_grid": (0, 2, 4, 2, 1, 1, 2, 1.0),
    "sq2_empty": (0, 2, 4, 3, 1, 1, 2, 0.0),
}


# fractional max-pooling, name: (kind, dim, nOut, nIn, batch, density, seed); pool size 2
FMP_CASES = {
    "fmp_po2": (0, 2, 7, 10, 3, 0.3, 11),
    "fmp_pd2": (1, 2, 6, 9, 3, 0.4, 12),
    "fmp_ro2": (2, 2, 5, 7, 3, 0.5, 13),
    "fmp_rd2": (3, 2, 8, 11, 2, 0.3, 14),
    "fmp_po3": (0, 3, 4, 6, 2, 0.2, 15),
    "fmp_rd3": (3, 3, 5, 7, 2, 0.2, 16),
    "fmp_pd1": (1, 1, 7, 10, 2, 0.6, 17),
}


def main():
    orc.build()
    ref = orc.Reference()
    out = {}
    # the hand-checkable 8x8 example: sites (5,5),(1,2),(2,2),(3,4),(6,1) with rows 1..5, background row 0
    keys = np.array([x * 8 + y for x, y in ((5, 5), (1, 2), (2, 2), (3, 4), (6, 1))], np.int64)
    a = ref.grid_rules(0, 2, 8, 6, 3, 1, 1, keys, np.arange(1, 6), [0, 5], [0])
    b = ref.grid_rules(0, 2, 6, 3, 2, 2, 1, a["out_keys"], a["out_rows"], a["out_off"], a["out_bg"])
    for tag, r in (("known8x8_conv", a), ("known8x8_pool", b)):
        for k, v in r.items():
            out["%s/%s" % (tag, k)] = np.asarray(v)
    out["known8x8_conv/in"] = keys
    for i, (name, (lat, dim, nOut, size, stride, mn, batch, dens)) in enumerate(sorted(CASES.items())):
        rng = np.random.default_rng(100 + i)
        nIn = size + (nOut - 1) * stride
        g = random_grids(rng, batch, dim, nIn, dens, triangular=(lat == 1))
        r = ref.grid_rules(lat, dim, nIn, nOut, size, stride, mn, *g)
        out[name + "/params"] = np.array([lat, dim, nIn, nOut, size, stride, mn], np.int32)
        for k, v in zip(("in_keys", "in_rows", "in_off", "in_bg"), g):
            out["%s/%s" % (name, k)] = v
        for k, v in r.items():
            out["%s/%s" % (name, k)] = np.asarray(v)
    for i, (name, (kind, dim, nOut, nIn, batch, dens, seed)) in enumerate(sorted(FMP_CASES.items())):
        rng = np.random.default_rng(300 + i)
        g = random_grids(rng, batch, dim, nIn, dens)
        r, ticks = ref.fmp_rules(kind, dim, nIn, nOut, 2, seed, *g)
        out[name + "/fmp_params"] = np.array([kind, dim, nIn, nOut, 2, seed], np.int64)
        out[name + "/ticks"] = ticks
        for k, v in zip(("in_keys", "in_rows", "in_off", "in_bg"), g):
            out["%s/%s" % (name, k)] = v
        for k, v in r.items():
            out["%s/%s" % (name, k)] = np.asarray(v)
    np.savez_compressed(os.path.join(HERE, "rules_golden.npz"), **out)
    print("wrote", len(out), "arrays")


if __name__ == "__main__":
    main()
