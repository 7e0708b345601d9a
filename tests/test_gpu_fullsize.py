"""Full-size runs of the benchmark configurations, checked through properties that do not need the
whole answer from the CPU: exact parity on seeded samples of query ids (walks are independent and
keyed by query id, so a sample is checked bit for bit), every transition is an edge the app may
take, -1 padding is a suffix, counters and histogram agree with the result, a second run is
identical.  The four configurations together take about 35 s on a B200 box (the graphs are generated
on the device) and up to 12 GB of host memory."""
import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import oracle_lib as O

pytestmark = pytest.mark.gpu


def _check(g, app, kw, starts, chunks, chunk_len, seed=1337):
    V, d = g.V, kw["d"]
    n = len(starts)
    eng = fw.Engine(g, 0)
    prm = fw.make_params(app, seed=seed, **kw)
    res, st, hist = eng.walk(prm, starts, want_hist=True)
    assert st.device_status == 0 and st.launches >= 1  # a hub-batched call is a series of launches
    # a second run gives the same walks
    res2, st2 = eng.walk(prm, starts)
    assert st2.steps == st.steps and st2.scanned == st.scanned
    assert np.array_equal(res, res2)
    del res2
    eng.close()
    # counters and histogram against the result itself
    assert np.array_equal(res[:, 0], starts)
    body = res[:, 1:]
    lengths = (body != -1).sum(axis=1)
    assert int(lengths.sum()) == st.steps
    assert np.array_equal(np.bincount(lengths, minlength=d + 1).astype(np.uint64), hist)
    # -1 padding is a suffix of every row
    assert ((body[:, :-1] != -1) | (body[:, 1:] == -1)).all()
    # sampled transitions are edges the app may take
    rng = np.random.default_rng(99)
    xadj, adj = g.xadj, g.adj
    weight, label = g.weight, g.label
    rows = rng.integers(0, n, 30000)
    cols = rng.integers(0, d, 30000)
    seen = 0
    for i, k in zip(rows.tolist(), cols.tolist()):
        v, x = int(res[i, k]), int(res[i, k + 1])
        if x == -1:
            continue
        b, e = int(xadj[v]), int(xadj[v + 1])
        j = b + int(np.searchsorted(adj[b:e], x))
        assert j < e and adj[j] == x, "walk %d step %d: %d -> %d is not an edge" % (i, k, v, x)
        if app == fw.APP_METAPATH:
            assert label[j] == kw["schema"][k % len(kw["schema"])]
        else:
            assert weight[j] > 0.0
        seen += 1
    assert seen > 100
    # exact parity on contiguous chunks of query ids
    scanned = 0
    for off in rng.integers(0, max(1, n - chunk_len), chunks).tolist():
        sl = slice(off, off + chunk_len)
        ref, _, sc, _ = O.walk(xadj, adj, weight, label, app, starts[sl], seed=seed, query_id_base=off, **kw)
        assert np.array_equal(res[sl], ref), "chunk at %d differs" % off
        scanned += sc
    assert scanned > 0
    return st


def test_config2_deepwalk_all_vertices():
    g = fw.rmat(22, 16 << 22, weight_range=(0.0, 1.0), device=0)
    st = _check(g, fw.APP_DEEPWALK, dict(d=80), np.arange(g.V, dtype=np.int32), chunks=32, chunk_len=256)
    assert st.steps > 10 ** 8
    g.close()


def test_config3_ppr_uniform_starts():
    g = fw.rmat(24, 32 << 24, weight_range=(0.0, 1.0), device=0)
    starts = np.random.default_rng(4).integers(0, g.V, 10 ** 7).astype(np.int32)
    _check(g, fw.APP_PPR, dict(d=80, tp=0.2), starts, chunks=32, chunk_len=256)
    g.close()


def test_config4_node2vec_all_vertices():
    g = fw.rmat(23, 32 << 23, a=0.6, b=0.19, c=0.19, weight_range=(1.0, 5.0), device=0)
    _check(g, fw.APP_NODE2VEC, dict(d=80, p=2.0, q=0.5), np.arange(g.V, dtype=np.int32), chunks=16, chunk_len=64)
    g.close()


def test_config5_metapath_int64_offsets():
    g = fw.rmat(26, 16 << 26, weight_range=None, n_labels=5, xadj_bits=64, device=0)
    assert g.xadj.dtype == np.int64
    _check(g, fw.APP_METAPATH, dict(d=5, schema=[0, 1, 2, 3, 4]), np.arange(g.V, dtype=np.int32),
           chunks=32, chunk_len=256)
    g.close()
