"""ctypes access to the CPU golden walker (oracle/libfw_oracle.so) plus exact
transition laws computed with numpy.  Test-side only."""
import ctypes
import os

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
_lib = None


def lib():
    global _lib
    if _lib is None:
        L = ctypes.CDLL(os.path.join(ROOT, "oracle", "libfw_oracle.so"))
        L.fwo_exp_key.restype = ctypes.c_float
        L.fwo_exp_key.argtypes = [ctypes.c_uint32]
        L.fwo_tp_threshold.restype = ctypes.c_uint32
        L.fwo_tp_threshold.argtypes = [ctypes.c_double]
        vp, i64 = ctypes.c_void_p, ctypes.c_int64
        L.fwo_walk.argtypes = [i64, vp, ctypes.c_int, vp, vp, vp, ctypes.c_int, ctypes.c_int,
                               ctypes.c_double, ctypes.c_double, ctypes.c_double, vp, ctypes.c_int,
                               ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_int, vp, i64, vp, vp,
                               ctypes.c_int]
        _lib = L
    return _lib


def philox(ctr, key):
    c = (ctypes.c_uint32 * 4)(*ctr)
    k = (ctypes.c_uint32 * 2)(*key)
    o = (ctypes.c_uint32 * 4)()
    lib().fwo_philox4x32_10(c, k, o)
    return list(o)


def walk(xadj, adj, weight, label, app, starts, d=80, tp=0.2, p=2.0, q=0.5, schema=None,
         seed=1337, query_id_base=0, group_mode=64, threads=0, query_id_stride=1):
    """Returns (result[n, d+1] int32, steps, scanned, len_hist[d+1])."""
    xadj = np.ascontiguousarray(xadj)
    assert xadj.dtype in (np.dtype(np.uint32), np.dtype(np.int64))
    adj = np.ascontiguousarray(adj, dtype=np.int32)
    w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
    lb = None if label is None else np.ascontiguousarray(label, dtype=np.int32)
    sc = None if schema is None else np.ascontiguousarray(schema, dtype=np.int32)
    starts = np.ascontiguousarray(starts, dtype=np.int32)
    n = len(starts)
    out = np.empty((n, d + 1), dtype=np.int32)
    stats = np.zeros(d + 3, dtype=np.uint64)
    rc = lib().fwo_walk(len(xadj) - 1, xadj.ctypes.data, 64 if xadj.dtype == np.int64 else 32,
                        adj.ctypes.data, None if w is None else w.ctypes.data,
                        None if lb is None else lb.ctypes.data, app, d, tp, p, q,
                        None if sc is None else sc.ctypes.data, 0 if sc is None else len(sc),
                        seed, query_id_base, query_id_stride, group_mode, starts.ctypes.data, n, out.ctypes.data,
                        stats.ctypes.data, threads)
    if rc != 0:
        raise RuntimeError("fwo_walk failed: %d" % rc)
    return out, int(stats[0]), int(stats[1]), stats[2:].copy()


def graph_walk(g, app, starts, **kw):
    return walk(g.xadj, g.adj, g.weight, g.label, app, starts, **kw)


# ---- exact transition laws (the distributional ground truth) ----

def row(xadj, v):
    return int(xadj[v]), int(xadj[v + 1])


def exact_bias(xadj, adj, weight, label, app, cur, prev, k, p=2.0, q=0.5, schema=None):
    """Bias vector over the row of `cur` at step k (0-based) coming from `prev` (-1: none)."""
    b, e = row(xadj, cur)
    if app == 3:
        return (label[b:e] == schema[k % len(schema)]).astype(np.float64)
    w = np.maximum(weight[b:e].astype(np.float64), 0.0)
    if app == 2 and prev >= 0:
        pb, pe = row(xadj, prev)
        prow = adj[pb:pe]
        nb = adj[b:e]
        is_prev = nb == prev
        linked = np.isin(nb, prow)
        w = np.where(is_prev, w / p, np.where(linked, w, w / q))
    return w


def chi_square_transitions(xadj, adj, weight, label, app, walks, min_expected=5.0, **kw):
    """Pooled Pearson chi-square of observed next-vertex counts against the exact law,
    conditioned on the state (cur, prev for node2vec, step class for MetaPath).
    Returns (chi2, dof, p_value)."""
    from scipy import stats as sps
    schema = kw.get("schema")
    counts = {}
    n, D = walks.shape
    for i in range(n):
        rowv = walks[i]
        for k in range(D - 1):
            nxt = rowv[k + 1]
            if nxt < 0:
                break
            cur = int(rowv[k])
            prev = int(rowv[k - 1]) if k > 0 else -1
            if app == 2:
                state = (cur, prev, 0)
            elif app == 3:
                state = (cur, -1, k % len(schema))
            else:
                state = (cur, -1, 0)
            counts.setdefault(state, {}).setdefault(int(nxt), 0)
            counts[state][int(nxt)] += 1
    chi2, dof = 0.0, 0
    for (cur, prev, kk), obs in counts.items():
        bias = exact_bias(xadj, adj, weight, label, app, cur, prev, kk, kw.get("p", 2.0),
                          kw.get("q", 0.5), schema)
        b, e = row(xadj, cur)
        nb = adj[b:e]
        total = sum(obs.values())
        tot_bias = bias.sum()
        assert tot_bias > 0
        # merge duplicate neighbour ids (multi-edges) into one cell
        cells = {}
        for x, bb in zip(nb.tolist(), bias.tolist()):
            cells[x] = cells.get(x, 0.0) + bb
        for x in obs:
            assert cells.get(x, 0.0) > 0.0, "sampled an edge of zero bias"
        exp = np.array([total * bb / tot_bias for bb in cells.values()])
        ob = np.array([obs.get(x, 0) for x in cells.keys()], dtype=np.float64)
        big = exp >= min_expected
        if big.sum() < 1:
            continue
        e_big, o_big = exp[big], ob[big]
        e_rest, o_rest = exp[~big].sum(), ob[~big].sum()
        if e_rest >= min_expected:
            e_big = np.append(e_big, e_rest)
            o_big = np.append(o_big, o_rest)
        elif e_rest > 0:
            e_big[-1] += e_rest
            o_big[-1] += o_rest
        if len(e_big) < 2:
            continue
        chi2 += float(((o_big - e_big) ** 2 / e_big).sum())
        dof += len(e_big) - 1
    pval = float(sps.chi2.sf(chi2, dof)) if dof > 0 else 1.0
    return chi2, dof, pval


def chi_square_state(xadj, adj, weight, label, app, cur, prev, k, nexts, min_expected=5.0, **kw):
    """Pearson chi-square of the observed next vertices `nexts` (one per visit of the state
    cur / prev / step k) against the exact law of that state; vectorised, for states visited
    millions of times (hub rows).  Cells below `min_expected` are pooled.  Returns (chi2, dof)."""
    bias = exact_bias(xadj, adj, weight, label, app, cur, prev, k, kw.get("p", 2.0), kw.get("q", 0.5),
                      kw.get("schema"))
    b, e = row(xadj, cur)
    ids, inv = np.unique(adj[b:e], return_inverse=True)          # parallel edges share a cell
    cell_bias = np.bincount(inv, weights=bias, minlength=len(ids))
    nexts = np.asarray(nexts)
    pos = np.minimum(np.searchsorted(ids, nexts), len(ids) - 1)
    assert (ids[pos] == nexts).all(), "sampled a vertex outside the row"
    obs = np.bincount(pos, minlength=len(ids)).astype(np.float64)
    assert (obs[cell_bias <= 0] == 0).all(), "sampled an edge of zero bias"
    keep = cell_bias > 0
    exp = len(nexts) * cell_bias[keep] / cell_bias[keep].sum()
    obs = obs[keep]
    big = exp >= min_expected
    e_big, o_big = exp[big], obs[big]
    if (~big).any():
        e_big = np.append(e_big, exp[~big].sum())
        o_big = np.append(o_big, obs[~big].sum())
    if len(e_big) < 2:
        return 0.0, 0
    return float(((o_big - e_big) ** 2 / e_big).sum()), len(e_big) - 1


def chi_square_pvalue(chi2, dof):
    from scipy import stats as sps
    return float(sps.chi2.sf(chi2, dof)) if dof > 0 else 1.0


def length_agreement(la, lb, d, family_level=0.01):
    """Two samples of walk lengths (same size): per-bin z-scores of the two histograms over the
    bins that hold at least 20 walks together, the 3-sigma reading of the criterion, and the
    threshold that keeps the family-wise false-alarm rate of `family_level` over those K bins
    (Bonferroni: z* = Phi^-1(1 - level / 2K); 3.0 when that is lower).  Returns a dict."""
    from scipy import stats as sps
    n = len(la)
    assert len(lb) == n
    ha = np.bincount(la, minlength=d + 1).astype(np.float64)
    hb = np.bincount(lb, minlength=d + 1).astype(np.float64)
    pooled = (ha + hb) / (2.0 * n)
    sigma = np.sqrt(pooled * (1 - pooled) * 2.0 / n)
    big = (ha + hb) >= 20
    z = (ha[big] - hb[big]) / n / sigma[big]
    K = int(big.sum())
    zstar = max(3.0, float(sps.norm.isf(family_level / (2.0 * max(K, 1)))))
    mean_z = abs(la.mean() - lb.mean()) / (np.sqrt((la.var() + lb.var()) / n) + 1e-300)
    return {"bins": K, "max_abs_z": float(np.abs(z).max()) if K else 0.0, "threshold": zstar,
            "beyond_3_sigma": int((np.abs(z) > 3.0).sum()), "mean_z": float(mean_z)}
