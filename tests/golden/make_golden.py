"""Regenerates tests/golden/config1_walks.npz from the CPU golden walker.

The reference cannot produce golden vectors (it has no CPU path, no tests, and its walks are
not reproducible), so these fixtures are outputs of oracle/fw_oracle.c on the config-1 graph
(7,115 vertices, 103,689 R-MAT edges, 100 seeded starts, d = 80; MetaPath d = 5).  They pin
the oracle and the graph generator against drift and give the GPU tests a file to compare with.

    python tests/golden/make_golden.py
"""
import hashlib
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

import graphs  # noqa: E402
import oracle_lib as O  # noqa: E402

CASES = [("deepwalk", 0, dict(d=80)), ("ppr", 1, dict(d=80, tp=0.2)),
         ("node2vec", 2, dict(d=80, p=2.0, q=0.5)), ("metapath", 3, dict(d=5, schema=[0, 1, 2, 3, 4]))]


def graph_digest(g):
    h = hashlib.sha256()
    for a in (g.xadj, g.adj, g.weight, g.label):
        h.update(np.ascontiguousarray(a).tobytes())
    return h.hexdigest()


def main():
    g = graphs.config1()
    starts = graphs.config1_starts()
    out = {"starts": starts, "graph_sha256": np.array(graph_digest(g))}
    for name, app, kw in CASES:
        for mode in (1, 64):
            res, steps, scanned, hist = O.graph_walk(g, app, starts, seed=1337, group_mode=mode, **kw)
            out["%s_g%d" % (name, mode)] = res
            out["%s_g%d_stats" % (name, mode)] = np.array([steps, scanned], dtype=np.uint64)
    np.savez_compressed(os.path.join(HERE, "config1_walks.npz"), **out)
    print("wrote", os.path.join(HERE, "config1_walks.npz"))


if __name__ == "__main__":
    main()
