"""Cross-check against the reference's own CUDA walker (unmodified sources rebuilt for sm_100
by oracle/build_ref.sh into oracle/_ref/ref_walk) on the same graph and start vertices:
its per-vertex transition frequencies and ours must both follow each app's exact weighted
transition law (chi-square, p > 0.001), and the walk-length distributions must agree.  The
reference is not reproducible run to run, so nothing here is bit-exact.

Walk lengths: per-bin z-scores of the two length histograms over the K bins that hold at
least 20 walks.  "Within 3 sigma" is applied per bin when it is a family-wise statement too
(few bins); with K bins and a fresh reference draw per run a bare 3-sigma rule on every bin
would fail a sound pair in about 0.27 % x K of the runs, so the bound is the one that keeps
the family-wise false-alarm rate at 1 %: z* = max(3, Phi^-1(1 - 0.005 / K)), i.e. 3.0 up to
4 bins, 3.5 at 20, 3.8 at 80.  The observed maximum and the number of bins beyond 3 sigma
are written into the run's record.

Three graphs: the config-1 graph (rows up to about a thousand neighbours: the reference's
warp sampler), a 100,000-leaf star with weights over two decades (its block sampler,
include/sampler.cuh:87-127, against this engine's staged ring sweep and its shared-row path),
and an R-MAT scale-16 graph whose hubs exceed 1,024 neighbours (both samplers mixed)."""
import json
import os
import subprocess

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs
import oracle_lib as O
from conftest import REPORT_LINES

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "oracle", "_ref", "ref_walk")
needs_ref = pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref/ref_walk has not been built")

CASES = [
    ("deepwalk", fw.APP_DEEPWALK, dict(d=80), 60000),
    ("ppr", fw.APP_PPR, dict(d=80, tp=0.2), 1500000),
    ("node2vec", fw.APP_NODE2VEC, dict(d=80, p=2.0, q=0.5), 60000),
    ("metapath", fw.APP_METAPATH, dict(d=5, schema=[0, 1, 2, 3, 4]), 200000),
]


def run_reference(tmp_path, prefix, name, kw, starts):
    sp = str(tmp_path / ("starts_%s.bin" % name))
    out = str(tmp_path / ("ref_%s.bin" % name))
    starts.tofile(sp)
    cmd = [REF, prefix, name, str(kw["d"]), sp, str(len(starts)), out,
           str(kw.get("tp", 0.2)), str(kw.get("p", 2.0)), str(kw.get("q", 0.5))]
    if "schema" in kw:
        cmd.append(",".join(str(x) for x in kw["schema"]))
    res = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-2000:] + res.stderr[-2000:]
    info = json.loads([ln for ln in res.stdout.splitlines() if ln.startswith("REFJSON ")][-1][8:])
    walks = np.fromfile(out, dtype=np.int32).reshape(len(starts), kw["d"] + 1)
    os.remove(out)
    return walks, info


def lengths(walks):
    return (walks[:, 1:] >= 0).sum(axis=1)


def check_lengths(tag, name, ref_walks, ours, n, d):
    """Under PPR the reference truncates the walks still in flight when its blocks run out of
    queries (its stop test also fires for empty slots and ends the block early,
    include/walker.cuh:1422-1431).  A walk of up to 80 rounds can still be in flight about a
    million claims after its own, so PPR compares only the first fifth of a long id range."""
    keep = n // 5 if name == "ppr" else n * 3 // 4
    r = O.length_agreement(lengths(ref_walks[:keep]), lengths(ours[:keep]), d)
    REPORT_LINES.append("walk lengths vs reference, %s %s: %d walks, %d bins, max|z| %.2f (bound %.2f), "
                        "%d bins beyond 3 sigma, mean z %.2f" % (tag, name, keep, r["bins"], r["max_abs_z"],
                                                                 r["threshold"], r["beyond_3_sigma"], r["mean_z"]))
    assert r["max_abs_z"] < r["threshold"], (tag, name, r)
    # the reference's walks differ from run to run, so this is a fresh draw every time: 4 sigma
    # (6e-5 two-sided) keeps a sound pair from failing once in a few hundred runs, as 3 sigma did,
    # while a 2 % shift of the mean length would still be a 6 sigma event
    assert r["mean_z"] < 4.0, (tag, name, r)


def engine_walks(arrs_or_graph, app, kw, starts, sharing=-1):
    g = arrs_or_graph if isinstance(arrs_or_graph, fw.Graph) else \
        fw.Graph.from_arrays(arrs_or_graph["xadj"], arrs_or_graph["adj"], arrs_or_graph["weight"], arrs_or_graph["label"])
    eng = fw.Engine(g, 0)
    eng.set_sharing(sharing)
    out, st = eng.walk(fw.make_params(app, **kw), starts)
    eng.close()
    assert st.device_status == 0
    return out


@needs_ref
@pytest.mark.parametrize("name,app,kw,n", CASES)
def test_same_law_as_reference(tmp_path, name, app, kw, n):
    g = graphs.config1()
    prefix = str(tmp_path / "cfg1")
    g.save(prefix)
    # starts drawn from a small pool of non-dead-end vertices, so that every visited state
    # collects enough transitions for the chi-square cells
    rng = np.random.default_rng(17)
    deg = np.diff(g.xadj.astype(np.int64))
    pool = rng.choice(np.nonzero(deg >= 8)[0], size=48, replace=False)
    starts = pool[rng.integers(0, len(pool), n)].astype(np.int32)
    ref_walks, info = run_reference(tmp_path, prefix, name, kw, starts)
    ours = engine_walks(g, app, kw, starts)
    assert (ref_walks[:, 0] == starts).all() and (ours[:, 0] == starts).all()
    law_kw = {k: v for k, v in kw.items() if k in ("p", "q", "schema")}
    m = 20000  # walks fed to the (python) transition counter
    for label, walks in (("reference", ref_walks), ("ours", ours)):
        chi2, dof, pval = O.chi_square_transitions(g.xadj, g.adj, g.weight, g.label, app, walks[:m], **law_kw)
        REPORT_LINES.append("transitions, config-1 %s, %s: chi2 %.0f on %d dof, p = %.3f" % (name, label, chi2, dof, pval))
        assert dof > 50 and pval > 0.001, (label, chi2, dof, pval)
    check_lengths("config-1", name, ref_walks, ours, n, kw["d"])


def hub_law(tag, arrs, app, kw, arms, state_of):
    """Chi-square of every arm's transitions out of the states `state_of(walks)` yields
    (cur, prev, step, next-vertex array) against the exact law."""
    law_kw = {k: v for k, v in kw.items() if k in ("p", "q", "schema")}
    for label, walks in arms:
        chi2 = dof = 0
        for cur, prev, k, nexts in state_of(walks):
            c, f = O.chi_square_state(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], app, cur, prev, k,
                                      nexts, **law_kw)
            chi2 += c
            dof += f
        pval = O.chi_square_pvalue(chi2, dof)
        REPORT_LINES.append("transitions, %s, %s: chi2 %.0f on %d dof, p = %.3f" % (tag, label, chi2, dof, pval))
        assert dof > 50 and pval > 0.001, (tag, label, chi2, dof, pval)


def star_two_decades():
    arrs = graphs.star()
    rng = np.random.default_rng(23)
    arrs["weight"][:100000] = (10.0 ** rng.uniform(-1.3, 0.7, 100000)).astype(np.float32)
    arrs["label"][:100000] = np.arange(100000) % 5
    return arrs


@needs_ref
@pytest.mark.parametrize("name,app,kw,n", [
    ("deepwalk", fw.APP_DEEPWALK, dict(d=1), 2000000),
    ("ppr", fw.APP_PPR, dict(d=6, tp=0.2), 1000000),
    ("metapath", fw.APP_METAPATH, dict(d=5, schema=[0, 1, 2, 3, 4]), 1000000),
    ("node2vec", fw.APP_NODE2VEC, dict(d=2, p=2.0, q=0.5), 4000000),
])
def test_star_hub_law_as_reference(tmp_path, name, app, kw, n):
    """The hub row of 100,000 neighbours, weights over two decades: the reference samples it with
    its block sampler, this engine with the staged ring sweep of one warp (sharing 0) and with the
    row shared between the warps of a CTA (sharing 1).  All three must follow the exact law of the
    hub's transitions; node2vec arrives at the hub from a leaf, so its p/q law over the row is tested."""
    arrs = star_two_decades()
    g = fw.Graph.from_arrays(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"])
    prefix = str(tmp_path / "star")
    g.save(prefix)
    if app == fw.APP_NODE2VEC:
        deg = np.diff(arrs["xadj"].astype(np.int64))
        leaves = np.nonzero(deg[1:] == 3)[0][:2] + 1   # two leaves with the hub and two more neighbours
        starts = leaves[np.arange(n) % 2].astype(np.int32)

        def state_of(walks):
            for leaf in leaves:
                sel = (walks[:, 0] == leaf) & (walks[:, 1] == 0) & (walks[:, 2] >= 0)
                yield 0, int(leaf), 1, walks[sel, 2]
    else:
        starts = np.zeros(n, dtype=np.int32)

        def state_of(walks):
            yield 0, -1, 0, walks[walks[:, 1] >= 0, 1]
    ref_walks, info = run_reference(tmp_path, prefix, name, kw, starts)
    arms = [("reference", ref_walks)]
    for sharing in (0, 1):
        arms.append(("ours sharing=%d" % sharing, engine_walks(g, app, kw, starts, sharing)))
    hub_law("star " + name, arrs, app, kw, arms, state_of)
    if name in ("ppr", "metapath"):
        check_lengths("star", name, ref_walks, arms[1][1], n, kw["d"])


@needs_ref
@pytest.mark.parametrize("name,app,kw", [
    ("deepwalk", fw.APP_DEEPWALK, dict(d=3)),
    ("ppr", fw.APP_PPR, dict(d=8, tp=0.2)),
    ("node2vec", fw.APP_NODE2VEC, dict(d=3, p=2.0, q=0.5)),
    ("metapath", fw.APP_METAPATH, dict(d=5, schema=[0, 1, 2, 3, 4])),
])
def test_rmat16_hub_law_as_reference(tmp_path, name, app, kw):
    """R-MAT scale 16, edge factor 16: walks started on the hubs of more than 1,024 neighbours.
    First-step transitions out of every hub and, for the second step, out of the most visited
    (previous, current) pairs -- node2vec's law with a hub as the previous vertex."""
    g = fw.rmat(16, 16 << 16, weight_range=(0.0, 1.0), n_labels=5)
    arrs = dict(xadj=g.xadj.copy(), adj=g.adj.copy(), weight=g.weight.copy(), label=g.label.copy())
    prefix = str(tmp_path / "r16")
    g.save(prefix)
    deg = np.diff(arrs["xadj"].astype(np.int64))
    hubs = np.argsort(-deg)[:40]
    hubs = hubs[deg[hubs] > 1024][::6][:6]          # six hubs spread over the degrees above 1,024
    assert len(hubs) >= 3 and deg[hubs].min() > 1024
    n = 900000
    starts = hubs[np.arange(n) % len(hubs)].astype(np.int32)

    def state_of(walks):
        for h in hubs:
            sel = (walks[:, 0] == h) & (walks[:, 1] >= 0)
            yield int(h), -1, 0, walks[sel, 1]
        two = walks[walks[:, 2] >= 0]
        pairs, counts = np.unique(two[:, :2], axis=0, return_counts=True)
        for j in np.argsort(-counts)[:60]:
            prev, cur = int(pairs[j, 0]), int(pairs[j, 1])
            sel = (two[:, 0] == prev) & (two[:, 1] == cur)
            yield cur, prev, 1, two[sel, 2]
    ref_walks, info = run_reference(tmp_path, prefix, name, kw, starts)
    arms = [("reference", ref_walks)]
    for sharing in (0, 1):
        arms.append(("ours sharing=%d" % sharing, engine_walks(g, app, kw, starts, sharing)))
    hub_law("rmat16 " + name, arrs, app, kw, arms, state_of)
    check_lengths("rmat16", name, ref_walks, arms[1][1], n, kw["d"])
