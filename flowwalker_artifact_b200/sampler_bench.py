"""Sampler micro-benchmark: neighbours per second against row length, on graphs whose rows all
have the same degree (the role of the reference's TestSampler.out, src/sampler_test.cu:714-916,
which times its samplers over 2 GiB of synthetic weights and never checks a result).  Every
timed walk goes through the C ABI; use the parity tests for correctness.

    python -m flowwalker_artifact_b200.sampler_bench [--app deepwalk] [--degrees 16,128,1024,8192,65536]
"""
import argparse
import json

import numpy as np

from . import _binding as fw

APPS = {"deepwalk": 0, "ppr": 1, "node2vec": 2, "metapath": 3}


def regular_graph(degree, edges=1 << 26, seed=1):
    """V = edges/degree vertices, each with `degree` sorted random neighbours (duplicates possible)."""
    V = max(edges // degree, 2)
    rng = np.random.default_rng(seed)
    xadj = (np.arange(V + 1, dtype=np.int64) * degree).astype(np.uint32)
    adj = rng.integers(0, V, size=(V, degree), dtype=np.int32)
    adj.sort(axis=1)
    return fw.Graph.from_arrays(xadj, adj.reshape(-1), rng.random(V * degree, dtype=np.float32),
                                rng.integers(0, 5, V * degree).astype(np.int32)), V


def main():
    import torch
    ap = argparse.ArgumentParser()
    ap.add_argument("--app", default="deepwalk", choices=list(APPS))
    ap.add_argument("--degrees", default="16,128,1024,8192,65536")
    ap.add_argument("--d", type=int, default=40)
    ap.add_argument("--group", type=int, default=0)
    ap.add_argument("--edges", type=int, default=1 << 26,
                    help="edges of each graph (2^26 = 268 MB of weights: twice the L2; 2^24 stays L2-resident)")
    ap.add_argument("--work", type=float, default=0.0,
                    help="neighbours to scan per launch (default 4e11; a small value keeps instrumented ncu captures short)")
    args = ap.parse_args()
    for degree in [int(x) for x in args.degrees.split(",")]:
        g, V = regular_graph(degree, edges=args.edges)
        eng = fw.Engine(g, 0)
        target = args.work or (4e11 if degree >= 64 else 5e10)
        n = int(min(max(target / (degree * args.d), 20000), 8e6))
        starts = torch.from_numpy(np.random.default_rng(2).integers(0, V, n).astype(np.int32)).cuda()
        res = torch.empty((n, args.d + 1), dtype=torch.int32, device="cuda")
        prm = fw.make_params(APPS[args.app], d=args.d, group_mode=args.group,
                             schema=[0, 1, 2, 3, 4] if args.app == "metapath" else None)
        torch.cuda.synchronize()
        eng.walk_device(prm, starts.data_ptr(), n, res.data_ptr())          # warm-up
        st = eng.walk_device(prm, starts.data_ptr(), n, res.data_ptr())
        print(json.dumps({"app": args.app, "degree": degree, "edges": args.edges, "queries": n, "steps": st.steps,
                          "kernel_ms": st.device_ms, "steps_per_s": st.steps / (st.device_ms * 1e-3),
                          "neighbours_per_s": st.scanned / (st.device_ms * 1e-3)}), flush=True)
        eng.close()
        g.close()


if __name__ == "__main__":
    main()
