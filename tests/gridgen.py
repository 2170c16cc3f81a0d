"""Random sparse grids for rule-construction tests (test infrastructure)."""
import numpy as np


def random_grids(rng, batch, dim, nIn, density, triangular=False, with_bg=True, first_row=0):
    """-> keys(int64), rows(int32), off, bg in the flat protocol of grid_rules.
    Rows are numbered like Picture::codifyInputData does: per sample the background row
    first (when with_bg), then the sites in a random insertion order."""
    keys, rows, off, bg = [], [], [0], []
    row = first_row
    cells = nIn ** dim
    allk = np.arange(cells, dtype=np.int64)
    if triangular:
        c = np.stack(np.unravel_index(allk, (nIn,) * dim), 0)
        allk = allk[c.sum(0) < nIn]
    for b in range(batch):
        d = density if np.isscalar(density) else density[b % len(density)]
        m = rng.random(len(allk)) < d
        k = allk[m]
        rng.shuffle(k)
        if with_bg:
            bg.append(row)
            row += 1
        else:
            bg.append(-1)
        keys.extend(k.tolist())
        rows.extend(range(row, row + len(k)))
        row += len(k)
        off.append(len(keys))
    return (np.array(keys, np.int64), np.array(rows, np.int32), np.array(off, np.int32), np.array(bg, np.int32))
