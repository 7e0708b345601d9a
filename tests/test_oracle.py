"""CPU tests of the golden walker: known-answer vectors, committed fixtures, sampling law."""
import os

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs
import oracle_lib as O

GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "config1_walks.npz")


def test_philox_known_answers():
    """Random123 kat_vectors for philox4x32-10."""
    assert O.philox([0, 0, 0, 0], [0, 0]) == [0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8]
    assert O.philox([0xffffffff] * 4, [0xffffffff] * 2) == [0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd]
    assert O.philox([0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344], [0xa4093822, 0x299f31d0]) == \
        [0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1]


def test_exp_key_is_exponential_and_precise():
    L = O.lib()
    # structure: leading-zero count is the integer part, exact -log2 at the cell edges
    assert L.fwo_exp_key(0x80000000) == pytest.approx(2.0 ** -33 * 0.7213475, rel=1e-4)
    assert L.fwo_exp_key(0x40000000) == pytest.approx(1.0, abs=1e-6)
    assert L.fwo_exp_key(1) == pytest.approx(31.0, abs=1e-5)
    assert L.fwo_exp_key(0) == pytest.approx(32.0, abs=1e-5)
    xs = np.random.default_rng(0).integers(0, 2 ** 32, 200000, dtype=np.uint64)
    e = np.array([L.fwo_exp_key(int(x)) for x in xs], dtype=np.float64) * np.log(2.0)
    assert (e > 0).all()
    assert abs(e.mean() - 1.0) < 4 / np.sqrt(len(e))
    assert abs((e ** 2).mean() - 2.0) < 4 * np.sqrt(20.0 / len(e))
    # against the closed form -log2(1 - m/2) + g on the g = 0 cell
    for x in (0x80000001, 0x80001234, 0x9abcdef0, 0xc0000000, 0xffffffff):
        m = ((x << 1) & 0xffffffff) / 2.0 ** 32 + 2.0 ** -33
        assert L.fwo_exp_key(x) == pytest.approx(-np.log2(1 - m / 2), rel=2e-5)


def test_tp_threshold():
    L = O.lib()
    assert L.fwo_tp_threshold(0.0) == 0 and L.fwo_tp_threshold(-1.0) == 0
    assert L.fwo_tp_threshold(1.0) == 0xFFFFFFFF and L.fwo_tp_threshold(0.5) == 0x80000000


def test_golden_fixtures():
    gold = np.load(GOLD)
    g = graphs.config1()
    import hashlib
    h = hashlib.sha256()
    for a in (g.xadj, g.adj, g.weight, g.label):
        h.update(np.ascontiguousarray(a).tobytes())
    assert h.hexdigest() == str(gold["graph_sha256"]), "R-MAT generator output changed"
    starts = graphs.config1_starts()
    assert (starts == gold["starts"]).all()
    cases = [("deepwalk", 0, dict(d=80)), ("ppr", 1, dict(d=80, tp=0.2)),
             ("node2vec", 2, dict(d=80, p=2.0, q=0.5)), ("metapath", 3, dict(d=5, schema=[0, 1, 2, 3, 4]))]
    for name, app, kw in cases:
        for mode in (1, 64):
            res, steps, scanned, _ = O.graph_walk(g, app, starts, seed=1337, group_mode=mode, **kw)
            assert (res == gold["%s_g%d" % (name, mode)]).all(), (name, mode)
            assert [steps, scanned] == gold["%s_g%d_stats" % (name, mode)].tolist()


def _small_graph():
    return fw.rmat(8, 3000, weight_range=(1.0, 5.0), n_labels=5)


@pytest.mark.parametrize("mode", [1, 64])
@pytest.mark.parametrize("app,kw", [(0, dict(d=8)), (1, dict(d=8, tp=0.2)), (2, dict(d=8, p=2.0, q=0.5)),
                                    (2, dict(d=8, p=0.25, q=4.0)), (3, dict(d=5, schema=[0, 1, 2, 3, 4])),
                                    (3, dict(d=6, schema=[2, 2, 0]))])
def test_transition_law_chi_square(app, kw, mode):
    """Per-vertex transition frequencies against the exact weighted law, p > 0.001."""
    g = _small_graph()
    starts = np.random.default_rng(4).integers(0, g.V, 30000).astype(np.int32)
    res, steps, _, _ = O.graph_walk(g, app, starts, group_mode=mode, seed=2024 + mode, **kw)
    law_kw = {k: v for k, v in kw.items() if k in ("p", "q", "schema")}
    chi2, dof, pval = O.chi_square_transitions(g.xadj, g.adj, g.weight, g.label, app, res, **law_kw)
    assert dof > 100 and pval > 0.001, (chi2, dof, pval)


def test_big_row_law_both_modes():
    """One row of 5,000 neighbours with weights over 3 decades: the strip sampler and the
    per-neighbour sampler both follow w/sum(w)."""
    from scipy import stats as sps
    rng = np.random.default_rng(3)
    deg = 5000
    w = (10.0 ** rng.uniform(-2, 1, deg)).astype(np.float32)
    xadj = np.concatenate([[0, 3], 3 + np.arange(1, 2) * deg, np.full(deg, 3 + deg)]).astype(np.uint32)
    # vertex 0: 3 edges (misaligns the hub row), vertex 1: the hub, the rest: dead ends
    adj = np.concatenate([[1, 1, 1], np.arange(2, deg + 2)]).astype(np.int32)
    weight = np.concatenate([[1, 1, 1], w]).astype(np.float32)
    V = deg + 2
    assert len(xadj) == V + 1
    n = 200000
    for mode in (1, 64):
        res, _, _, _ = O.walk(xadj, adj, weight, None, 0, np.ones(n, dtype=np.int32), d=1, group_mode=mode)
        obs = np.bincount(res[:, 1] - 2, minlength=deg).astype(np.float64)
        exp = n * w.astype(np.float64) / w.astype(np.float64).sum()
        order = np.argsort(exp)
        # pool the small cells into bins of expected count >= 20
        bins_o, bins_e, ao, ae = [], [], 0.0, 0.0
        for i in order:
            ao += obs[i]
            ae += exp[i]
            if ae >= 20:
                bins_o.append(ao)
                bins_e.append(ae)
                ao = ae = 0.0
        bins_e[-1] += ae
        bins_o[-1] += ao
        chi2 = float(((np.array(bins_o) - np.array(bins_e)) ** 2 / np.array(bins_e)).sum())
        pval = sps.chi2.sf(chi2, len(bins_e) - 1)
        assert pval > 0.001, (mode, chi2, len(bins_e), pval)


def test_ppr_length_law_within_3_sigma():
    """On a graph without dead ends the PPR walk length is min(Geom(tp), d)."""
    V, d, tp, n = 64, 80, 0.2, 200000
    rows = [np.setdiff1d(np.arange(V), [v]) for v in range(V)]
    g = graphs.from_rows(rows, V=V)
    starts = np.random.default_rng(1).integers(0, V, n).astype(np.int32)
    _, steps, _, hist = O.walk(g["xadj"], g["adj"], g["weight"], None, 1, starts, d=d, tp=tp)
    assert hist[0] == 0 and hist.sum() == n
    k = np.arange(1, d + 1)
    prob = tp * (1 - tp) ** (k - 1)
    prob[-1] = (1 - tp) ** (d - 1)
    exp = n * prob
    sigma = np.sqrt(n * prob * (1 - prob))
    big = exp >= 10
    z = (hist[1:][big].astype(np.float64) - exp[big]) / sigma[big]
    assert np.abs(z).max() < 4.0 and (np.abs(z) > 3.0).sum() <= 1, z
    assert abs(steps / n - (1 - (1 - tp) ** d) / tp) < 0.05


def test_edge_cases():
    arrs = graphs.ragged()
    xa = arrs["xadj"].astype(np.int64)
    deg = np.diff(xa)
    dead = int(np.nonzero(deg == 0)[0][0])
    res, steps, scanned, hist = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 0,
                                       np.array([dead], dtype=np.int32), d=5)
    assert res.tolist() == [[dead, -1, -1, -1, -1, -1]] and steps == 0 and scanned == 0 and hist[0] == 1
    # zero queries, zero steps
    res, steps, _, _ = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], None, 0, np.zeros(0, np.int32), d=3)
    assert res.shape == (0, 4) and steps == 0
    res, steps, _, _ = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], None, 0, np.array([5], np.int32), d=0)
    assert res.tolist() == [[5]] and steps == 0
    # never a zero- or negative-weight edge; 32- and 64-bit offsets agree
    starts = np.arange(arrs["n_rows"], dtype=np.int32)
    r32 = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 0, starts, d=6)[0]
    r64 = O.walk(xa, arrs["adj"], arrs["weight"], arrs["label"], 0, starts, d=6)[0]
    assert (r32 == r64).all()
    for row in r32:
        for k in range(6):
            if row[k + 1] < 0:
                break
            b, e = xa[row[k]], xa[row[k] + 1]
            hit = np.nonzero(arrs["adj"][b:e] == row[k + 1])[0]
            assert len(hit) and (arrs["weight"][b:e][hit] > 0).any()
    # a label that no edge of the row carries ends the walk
    nolabel = int(np.nonzero([np.all(arrs["label"][xa[v]:xa[v + 1]] == 9) and deg[v] > 0
                              for v in range(arrs["n_rows"])])[0][0])
    res = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 3,
                 np.array([nolabel], np.int32), d=5, schema=[0, 1, 2, 3, 4])[0]
    assert (res[0, 1:] == -1).all()
    # query ids key the stream: shards reproduce the full run
    a = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], None, 0, starts[:50], d=6, query_id_base=0)[0]
    b = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], None, 0, starts[50:], d=6, query_id_base=50)[0]
    assert (np.vstack([a, b]) == r32).all()


def test_hub_law_helpers_on_the_golden_walker():
    """The vectorised chi-square used for hub rows and the walk-length comparison, exercised on the
    golden walker itself: a 3,000-neighbour row with weights over two decades (DeepWalk and, arriving
    from a neighbour, node2vec), and two independent PPR runs whose lengths must agree."""
    rng = np.random.default_rng(3)
    V = 3001
    rows = [np.arange(1, V)] + [np.unique(np.concatenate([[0], rng.integers(1, V, 2)])) for _ in range(1, V)]
    arrs = graphs.from_rows(rows, V=V, rng=rng)
    arrs["weight"][:V - 1] = (10.0 ** rng.uniform(-1.3, 0.7, V - 1)).astype(np.float32)
    n = 300000
    walks = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 0, np.zeros(n, np.int32), d=1)[0]
    chi2, dof = O.chi_square_state(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 0, 0, -1, 0, walks[:, 1])
    assert dof > 2000 and O.chi_square_pvalue(chi2, dof) > 0.001
    # a wrong law (uniform weights) must be rejected by the same statistic
    chi2u, dofu = O.chi_square_state(arrs["xadj"], arrs["adj"], np.ones_like(arrs["weight"]), arrs["label"], 0, 0, -1,
                                     0, walks[:, 1])
    assert O.chi_square_pvalue(chi2u, dofu) < 1e-6
    leaf = 7
    w2 = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 2, np.full(n, leaf, np.int32), d=2,
                p=2.0, q=0.5)[0]
    sel = (w2[:, 1] == 0) & (w2[:, 2] >= 0)
    chi2, dof = O.chi_square_state(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], 2, 0, leaf, 1,
                                   w2[sel, 2], p=2.0, q=0.5)
    assert dof > 1000 and O.chi_square_pvalue(chi2, dof) > 0.001
    g = graphs.config1()
    starts = graphs.config1_starts(200000, seed=8)
    la = (O.graph_walk(g, 1, starts, d=80, tp=0.2, seed=1)[0][:, 1:] >= 0).sum(axis=1)
    lb = (O.graph_walk(g, 1, starts, d=80, tp=0.2, seed=2)[0][:, 1:] >= 0).sum(axis=1)
    r = O.length_agreement(la, lb, 80)
    assert r["bins"] > 10 and r["max_abs_z"] < r["threshold"] and 3.0 <= r["threshold"] < 4.0 and r["mean_z"] < 4.0
    shifted = O.length_agreement(la, np.minimum(lb + (np.arange(len(lb)) % 10 == 0), 80), 80)
    assert shifted["max_abs_z"] > shifted["threshold"]
