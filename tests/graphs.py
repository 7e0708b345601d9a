"""Seeded test graphs (numpy, host only)."""
import numpy as np

import flowwalker_artifact_b200 as fw


def config1():
    """Shape of BASELINE config 1: 7,115 vertices, 103,689 directed R-MAT edges,
    weights in [1,5), labels in {0..4}."""
    return fw.rmat(13, 0, a=0.57, b=0.19, c=0.19, seed=1, v_limit=7115, e_target=103689,
                   weight_range=(1.0, 5.0), weight_seed=2, n_labels=5, label_seed=3)


def config1_starts(n=100, V=7115, seed=4):
    return np.random.default_rng(seed).integers(0, V, n).astype(np.int32)


def from_rows(rows, V=None, rng=None, weight_range=(0.5, 2.0), n_labels=5, xadj_dtype=np.uint32):
    """rows: list of sorted neighbour-id lists.  Returns dict of CSR arrays."""
    rng = rng or np.random.default_rng(7)
    V = V or len(rows)
    deg = np.array([len(r) for r in rows] + [0] * (V - len(rows)), dtype=np.int64)
    xadj = np.concatenate([[0], np.cumsum(deg)]).astype(xadj_dtype)
    adj = np.concatenate([np.asarray(r, dtype=np.int32) for r in rows] + [np.zeros(0, np.int32)])
    E = len(adj)
    weight = rng.uniform(weight_range[0], weight_range[1], E).astype(np.float32)
    label = rng.integers(0, n_labels, E).astype(np.int32)
    return dict(xadj=xadj, adj=adj.astype(np.int32), weight=weight, label=label)


def ragged(xadj_dtype=np.uint32, seed=11):
    """Rows of every awkward length at every 16-byte misalignment, a hub, dead ends,
    an all-zero-weight row and a row whose labels never match."""
    rng = np.random.default_rng(seed)
    lengths = [1, 2, 3, 4, 5, 31, 32, 33, 63, 64, 65, 127, 128, 129, 511, 512, 513, 1023, 1024,
               1025, 2047, 2048, 2049, 4100]
    V = 6000
    rows = []
    for rep in range(4):
        for L in lengths:
            rows.append(np.sort(rng.choice(V, size=L, replace=False)))
            rows.append(np.sort(rng.choice(V, size=(rep + len(rows)) % 4, replace=False)))  # shifts alignment
    rows.append(np.sort(rng.choice(V, size=5500, replace=False)))   # hub
    rows.append(np.zeros(0, dtype=np.int64))                         # dead end
    zero_row = len(rows)
    rows.append(np.sort(rng.choice(V, size=40, replace=False)))     # all-zero weights
    nolabel_row = len(rows)
    rows.append(np.sort(rng.choice(V, size=77, replace=False)))     # label 9 only
    n_rows = len(rows)
    for v in range(n_rows, V):  # every other vertex leads back into the awkward rows
        rows.append(np.sort(rng.choice(n_rows, size=3, replace=False)))
    g = from_rows(rows, V=V, rng=rng, xadj_dtype=xadj_dtype)
    xa = g["xadj"].astype(np.int64)
    g["weight"][xa[zero_row]:xa[zero_row + 1]] = 0.0
    g["label"][xa[nolabel_row]:xa[nolabel_row + 1]] = 9
    # sprinkle zero and negative weights elsewhere
    idx = rng.choice(len(g["weight"]), size=len(g["weight"]) // 10, replace=False)
    g["weight"][idx[: len(idx) // 2]] = 0.0
    g["weight"][idx[len(idx) // 2:]] = -1.0
    g["n_rows"] = n_rows
    return g


def star(deg=100000, seed=5):
    """One hub pointing at `deg` leaves, every leaf pointing back at the hub and at a few leaves."""
    rng = np.random.default_rng(seed)
    V = deg + 1
    rows = [np.arange(1, V)]
    for v in range(1, V):
        extra = rng.integers(1, V, 2)
        rows.append(np.unique(np.concatenate([[0], extra[extra != v]])))
    return from_rows(rows, V=V, rng=rng)
