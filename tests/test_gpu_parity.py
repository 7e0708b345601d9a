"""Bit-exact parity of the CUDA engine (through the C ABI) with the CPU golden walker."""
import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs
import oracle_lib as O

pytestmark = pytest.mark.gpu

APPS = [
    (fw.APP_DEEPWALK, dict(d=80)),
    (fw.APP_PPR, dict(d=80, tp=0.2)),
    (fw.APP_NODE2VEC, dict(d=80, p=2.0, q=0.5)),
    (fw.APP_METAPATH, dict(d=5, schema=[0, 1, 2, 3, 4])),
]
MODES = [fw.GROUP_STRIP, fw.GROUP_EDGE]


def run_both(arrs, app, kw, starts, mode, seed=1337, base=0, sharing=-1, managed=False, hub=1):
    g = fw.Graph.from_arrays(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"])
    eng = fw.Engine(g, 0, managed=managed)
    eng.set_sharing(sharing)
    eng.set_hub_batching(hub)
    prm = fw.make_params(app, group_mode=mode, seed=seed, query_id_base=base, **kw)
    res, st, hist = eng.walk(prm, starts, want_hist=True)
    ref, steps, scanned, rhist = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], app,
                                        starts, seed=seed, query_id_base=base, group_mode=mode, **kw)
    eng.close()
    g.close()
    return res, st, hist, ref, steps, scanned, rhist


def assert_same(out):
    res, st, hist, ref, steps, scanned, rhist = out
    bad = np.nonzero((res != ref).any(axis=1))[0]
    assert len(bad) == 0, "walks differ, first at query %d:\n%s\n%s" % (bad[0], res[bad[0]], ref[bad[0]])
    assert st.steps == steps and st.scanned == scanned
    assert (hist == rhist).all()
    assert st.device_status == 0
    assert st.launches >= 1  # one kernel, or the series of launches of a hub-batched call


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("app,kw", APPS)
def test_config1(app, kw, mode):
    g = graphs.config1()
    arrs = dict(xadj=g.xadj.copy(), adj=g.adj.copy(), weight=g.weight.copy(), label=g.label.copy())
    assert_same(run_both(arrs, app, kw, graphs.config1_starts(), mode))


@pytest.mark.parametrize("bits", [32, 64])
@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("app,kw", APPS)
def test_ragged_rows(app, kw, mode, bits):
    arrs = graphs.ragged(np.uint32 if bits == 32 else np.int64)
    starts = np.concatenate([np.arange(arrs["n_rows"]), np.arange(arrs["n_rows"])]).astype(np.int32)
    kw = dict(kw)
    kw["d"] = min(kw["d"], 12)
    assert_same(run_both(arrs, app, kw, starts, mode, seed=99, base=1 << 33))


@pytest.mark.parametrize("mode", MODES)
@pytest.mark.parametrize("app,kw", APPS[:3])
def test_star_hub(app, kw, mode):
    arrs = graphs.star()
    starts = np.zeros(64, dtype=np.int32)
    kw = dict(kw)
    kw["d"] = 10
    assert_same(run_both(arrs, app, kw, starts, mode))


@pytest.mark.parametrize("app,d", [(fw.APP_DEEPWALK, 4095), (fw.APP_DEEPWALK, 4000), (fw.APP_NODE2VEC, 3800),
                                   (fw.APP_NODE2VEC, 4095), (fw.APP_PPR, 4096), (fw.APP_DEEPWALK, 9000)])
def test_long_walks_around_the_shared_memory_limits(app, d):
    """Walk lengths at which the length histogram plus the staging rings reach 48 KB of shared
    memory (the kernel's static part counts too) and at which the histogram leaves shared memory."""
    g = graphs.config1()
    arrs = dict(xadj=g.xadj.copy(), adj=g.adj.copy(), weight=g.weight.copy(), label=g.label.copy())
    kw = dict(d=d, tp=0.001) if app == fw.APP_PPR else dict(d=d)
    assert_same(run_both(arrs, app, kw, graphs.config1_starts(96, seed=d), fw.GROUP_STRIP))


@pytest.mark.parametrize("n", [3, 9, 64, 1000])
@pytest.mark.parametrize("app,kw", APPS + [(fw.APP_NODE2VEC, dict(d=80, p=0.25, q=4.0)),
                                          (fw.APP_NODE2VEC, dict(d=80, p=4.0, q=0.25))])
def test_star_hub_shared_between_warps(app, kw, n):
    """Rows of 100,000 edges with the block-granularity path forced on: warps that are out of
    queries take supergroups from the back of a posted row; the walks must not change.  With 3 or
    9 queries most warps of the CTA are idle from the start, with 1000 they become idle at the end."""
    arrs = graphs.star()
    arrs["label"][:100000] = np.arange(100000) % 5
    starts = np.zeros(n, dtype=np.int32)
    starts[1::2] = np.arange(1, n, 2) % 1000 + 1   # leaves lead straight back to the hub
    kw = dict(kw)
    kw["d"] = min(kw["d"], 10)
    assert_same(run_both(arrs, app, kw, starts, fw.GROUP_STRIP, seed=5, sharing=1))


@pytest.mark.parametrize("hub", [0, 1, 2])
@pytest.mark.parametrize("app,kw", APPS + [(fw.APP_METAPATH, dict(d=7, schema=[3, 3, 0])),
                                          (fw.APP_NODE2VEC, dict(d=80, p=0.25, q=4.0))])
def test_hub_batching_on_and_off(app, kw, hub):
    """Walkers that meet at a vertex of 1,024 or more neighbours share one sweep of its row (a walk
    call is then a series of launches); with it switched off every walker sweeps for itself in one
    kernel.  Both give the golden walker's walks: rows around the hub limit, a 100,000-leaf star
    where every walker is at the hub every other step, queries that start at hubs, PPR's stop test
    after a hub step, 32- and 64-bit offsets.  hub = 2 batches down to the last walker; hub = 1
    leaves the last few to one launch that does not batch (the default does the same on calls
    large enough to earn back the fixed cost of the series)."""
    arrs = graphs.ragged(np.int64 if app == fw.APP_PPR else np.uint32)
    starts = np.concatenate([np.arange(arrs["n_rows"])] * 3).astype(np.int32)
    kw2 = dict(kw)
    kw2["d"] = 15 if app != fw.APP_METAPATH else kw["d"]
    out = run_both(arrs, app, kw2, starts, fw.GROUP_STRIP, seed=21, base=7, hub=hub)
    assert_same(out)
    assert (out[1].launches == 1) == (hub == 0)
    star = graphs.star()
    star["label"][:100000] = np.arange(100000) % 5
    starts = np.zeros(3000, dtype=np.int32)
    starts[1::3] = np.arange(1, 3000, 3) % 1000 + 1
    out = run_both(star, app, kw2, starts, fw.GROUP_STRIP, seed=22, hub=hub)
    assert_same(out)
    assert (out[1].launches == 1) == (hub == 0)
    # d = 1: every walker that starts at the hub ends right after the hub step
    assert_same(run_both(star, app, dict(kw, d=1), np.zeros(100, dtype=np.int32), fw.GROUP_STRIP, hub=hub))


@pytest.mark.parametrize("app,kw", APPS)
def test_early_delivery_into_page_locked_memory(app, kw):
    """A hub-batched call whose result buffer is page-locked host memory may write the rows of
    ended walks to it round by round (deliver_kernel on a stream of its own) instead of copying the
    table after the last launch.  Same table every way, and the golden walker's: delivery to the
    last row (mode 1), delivery stopped and the table copied after all (mode 2), the engine's own
    choice (-1), no delivery (0); one batch and several (rows of the later batches start anywhere
    in the host table), the callee's buffer (fw_walk_batch), a caller's page-locked buffer at an
    odd offset (fw_walk_batch_into, fw_walk), pageable memory (nothing to deliver to), and rows too
    short to be delivered (MetaPath's 6 cells)."""
    import torch
    cases = []
    arrs = graphs.ragged()
    cases.append((arrs, np.concatenate([np.arange(arrs["n_rows"])] * 3).astype(np.int32), 33))
    star = graphs.star()
    star["label"][:100000] = np.arange(100000) % 5
    starts = np.zeros(3000, dtype=np.int32)
    starts[1::3] = np.arange(1, 3000, 3) % 1000 + 1
    cases.append((star, starts, 31))
    r = fw.rmat(16, 16 << 16, weight_range=(0.0, 1.0), n_labels=5)
    cases.append((dict(xadj=r.xadj.copy(), adj=r.adj.copy(), weight=r.weight.copy(), label=r.label.copy()),
                  np.arange(r.V, dtype=np.int32), 40))
    for arrs, starts, d in cases:
        kw2 = dict(kw, d=d if app != fw.APP_METAPATH else kw["d"])
        n, D = len(starts), kw2["d"] + 1
        g = fw.Graph.from_arrays(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"])
        eng = fw.Engine(g, 0)
        eng.set_hub_batching(1)
        prm = fw.make_params(app, seed=31, query_id_base=5, **kw2)
        ref, steps, _, _ = O.walk(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"], app, starts,
                                  seed=31, query_id_base=5, **kw2)
        launches = {}
        for mode in (1, 2, -1, 0):
            eng.set_early_delivery(mode)
            out, st = eng.walk_batch(prm, starts, batch_size=n)
            assert (out == ref).all() and st.steps == steps and st.device_status == 0
            launches[mode] = st.launches
            out, st = eng.walk_batch(prm, starts, batch_size=max(n // 3 - 7, 1))
            assert (out == ref).all() and st.steps == steps
            # a caller's page-locked buffer, the table 12 bytes off its start
            flat = torch.full((n * D + 8,), -9, dtype=torch.int32).pin_memory()
            table = flat[3:3 + n * D]
            st2 = fw.WalkStats()
            assert fw.lib().fw_walk_batch_into(eng._h, prm[0], starts.ctypes.data, n, n, 512, table.data_ptr(), st2, None) == 0
            assert (table.numpy().reshape(n, D) == ref).all()
            assert flat[:3].tolist() == [-9] * 3 and flat[3 + n * D:].tolist() == [-9] * 5
            flat.fill_(-9)
            st3 = fw.WalkStats()
            assert fw.lib().fw_walk(eng._h, prm[0], starts.ctypes.data, n, table.data_ptr(), st3, None) == 0
            assert (table.numpy().reshape(n, D) == ref).all()
            assert flat[:3].tolist() == [-9] * 3 and flat[3 + n * D:].tolist() == [-9] * 5
            if mode in (0, 1, 2):  # the engine's own choice depends on the clock
                assert st2.launches == launches[mode] and st3.launches == launches[mode]
        if D >= 32:  # the delivery launches are counted: one per round, and one more for the last rows
            assert launches[1] == launches[2] + 1 and launches[2] > launches[0] > 1
        else:
            assert launches[1] == launches[2] == launches[0] > 1
        assert launches[0] <= launches[-1] <= launches[1]
        # pageable memory: nothing the device could write to, one copy at the end
        eng.set_early_delivery(1)
        out, st = eng.walk(prm, starts)
        assert (out == ref).all() and st.launches == launches[0]
        # the same pageable array page-locked by the caller (cudaHostRegister): delivered to if the
        # device can address it, copied to otherwise; the same table either way
        own = np.full((n, D), -9, dtype=np.int32)
        rt = torch.cuda.cudart()
        assert int(rt.cudaHostRegister(own.ctypes.data, own.nbytes, 0)) == 0
        try:
            st4 = fw.WalkStats()
            assert fw.lib().fw_walk(eng._h, prm[0], starts.ctypes.data, n, own.ctypes.data, st4, None) == 0
            assert (own == ref).all() and st4.launches in (launches[0], launches[1])
        finally:
            rt.cudaHostUnregister(own.ctypes.data)
        eng.close()
        g.close()


@pytest.mark.parametrize("app,kw", APPS)
def test_rmat16_many_queries(app, kw):
    g = fw.rmat(16, 16 << 16, weight_range=(0.0, 1.0), n_labels=5)
    arrs = dict(xadj=g.xadj.copy(), adj=g.adj.copy(), weight=g.weight.copy(), label=g.label.copy())
    starts = np.arange(g.V, dtype=np.int32)
    kw = dict(kw)
    kw["d"] = min(kw["d"], 20)
    assert_same(run_both(arrs, app, kw, starts, fw.GROUP_STRIP))


def test_empty_and_bad_inputs():
    arrs = graphs.ragged()
    g = fw.Graph.from_arrays(arrs["xadj"], arrs["adj"], arrs["weight"], arrs["label"])
    eng = fw.Engine(g, 0)
    prm = fw.make_params(fw.APP_DEEPWALK, d=4)
    res, st = eng.walk(prm, np.zeros(0, dtype=np.int32))
    assert res.shape == (0, 5) and st.steps == 0 and st.launches == 0
    res, st = eng.walk(prm, np.array([-5, 10 ** 6, 3], dtype=np.int32))
    assert st.device_status & 1
    assert (res[0, 1:] == -1).all() and res[0, 0] == -5 and (res[1, 1:] == -1).all()
    res0, st0 = eng.walk(fw.make_params(fw.APP_DEEPWALK, d=0), np.array([3, 4], dtype=np.int32))
    assert res0.tolist() == [[3], [4]] and st0.steps == 0
    with pytest.raises(fw.FlowWalkerError):
        eng.walk(fw.make_params(fw.APP_METAPATH, d=5), np.array([1], dtype=np.int32))  # no schema
    with pytest.raises(fw.FlowWalkerError):
        eng.walk(fw.make_params(7, d=5), np.array([1], dtype=np.int32))
    eng.close()


def test_shards_union_equals_single_run():
    """Query ids key the random stream: two shards with their id bases reproduce the 1-GPU run."""
    g = graphs.config1()
    eng = fw.Engine(g, 0)
    starts = graphs.config1_starts(1000)
    full, _ = eng.walk(fw.make_params(fw.APP_DEEPWALK, d=40), starts)
    a, _ = eng.walk(fw.make_params(fw.APP_DEEPWALK, d=40, query_id_base=0), starts[:500])
    b, _ = eng.walk(fw.make_params(fw.APP_DEEPWALK, d=40, query_id_base=500), starts[500:])
    assert (np.vstack([a, b]) == full).all()
    # interleaved shards: rank r of 3 walks the ids r, r + 3, ... (query_id_stride)
    for r in range(3):
        part, _ = eng.walk(fw.make_params(fw.APP_DEEPWALK, d=40, query_id_base=r, query_id_stride=3), starts[r::3])
        assert (part == full[r::3]).all()
    strided, _ = eng.walk_batch(fw.make_params(fw.APP_DEEPWALK, d=40, query_id_base=1, query_id_stride=3),
                                starts[1::3], batch_size=100)
    assert (strided == full[1::3]).all()
    out, st = eng.walk_batch(fw.make_params(fw.APP_DEEPWALK, d=40), starts, batch_size=128)
    assert (out == full).all() and st.launches >= 8
    auto, st_auto = eng.walk_batch(fw.make_params(fw.APP_DEEPWALK, d=40), starts, batch_size=0)  # autobatch
    assert (auto == full).all() and st_auto.launches >= 1
    into = np.full((1000, 41), -9, dtype=np.int32)
    st2 = fw.WalkStats()
    prm = fw.make_params(fw.APP_DEEPWALK, d=40)
    rc = fw.lib().fw_walk_batch_into(eng._h, prm[0], starts.ctypes.data, 1000, 300, 512, into.ctypes.data, st2, None)
    assert rc == 0 and (into == full).all() and st2.launches >= 4 and st2.steps == st.steps
    eng.close()


def test_bounded_wait_reports_instead_of_hanging():
    """A wait that nothing completes runs out after its poll limit, sets the status word and
    leaves the context usable (the next walk still matches the golden walker)."""
    import ctypes
    L = fw.lib()
    status = ctypes.c_uint32(0)
    assert L.fw_selftest_wait_timeout(0, 2000, ctypes.byref(status)) == 0, L.fw_last_error()
    assert status.value == 4  # FW_STATUS_WAIT_TIMEOUT
    g = graphs.config1()
    arrs = dict(xadj=g.xadj.copy(), adj=g.adj.copy(), weight=g.weight.copy(), label=g.label.copy())
    assert_same(run_both(arrs, fw.APP_DEEPWALK, dict(d=20), graphs.config1_starts(), fw.GROUP_STRIP))


def _threshold_graph(rng, case):
    """Rows whose lengths sit around every dispatch threshold of the kernel; the other vertices
    are three-neighbour rows that lead back into them."""
    V = 9000
    marks = [1, 2, 5, 31, 32, 33, 120, 127, 128, 129, 131, 255, 256, 257, 500, 511, 512, 513, 1023, 1025,
             2047, 2048, 2049, 2100, 4095, 4096, 4100, 6000, 8191, 8200]
    degs = [int(rng.choice(marks)) for _ in range(300)] + [0] * 5
    if case % 3 == 0:
        degs += [8999, 7000]
    rng.shuffle(degs)
    n_rows = len(degs)
    rows = []
    for dg in degs:
        if case % 2 == 1:  # parallel edges, and rows that share many neighbours
            rows.append(np.sort(rng.integers(0, 4 * n_rows, size=dg)))
        else:
            rows.append(np.sort(rng.choice(V, size=dg, replace=False)))
    for v in range(n_rows, V):
        rows.append(np.sort(rng.choice(n_rows, size=3, replace=False)))
    g = graphs.from_rows(rows, V=V, rng=rng, weight_range=(0.05, 3.0),
                         xadj_dtype=np.uint32 if case % 2 else np.int64)
    if case % 4 >= 2:  # zero and negative weights
        idx = rng.choice(len(g["weight"]), size=len(g["weight"]) // 7, replace=False)
        g["weight"][idx[::2]] = 0.0
        g["weight"][idx[1::2]] = -2.0
    return g, n_rows


@pytest.mark.parametrize("case", range(10))
def test_random_graphs_all_apps(case):
    """Seeded random graphs: row lengths around 32 quads, two and three sub-blocks, one and several
    supergroups; parallel edges; zero and negative weights; p and q on both sides of 1; several
    stop probabilities and schemas; both offset widths; sharing on and off."""
    rng = np.random.default_rng(1000 + case)
    arrs, n_rows = _threshold_graph(rng, case)
    starts = rng.integers(0, n_rows, 600).astype(np.int32)
    p, q = [(2.0, 0.5), (0.25, 4.0), (1.0, 1.0), (0.5, 3.0), (4.0, 0.25)][case % 5]
    cases = [(fw.APP_DEEPWALK, dict(d=9)), (fw.APP_PPR, dict(d=30, tp=[0.05, 0.2, 0.6][case % 3])),
             (fw.APP_NODE2VEC, dict(d=9, p=p, q=q)),
             (fw.APP_METAPATH, dict(d=6, schema=[[0, 1, 2, 3, 4], [2, 2, 0], [4]][case % 3]))]
    for app, kw in cases:
        for mode in ((fw.GROUP_STRIP, fw.GROUP_EDGE) if case < 4 else (fw.GROUP_STRIP,)):
            assert_same(run_both(arrs, app, kw, starts, mode, seed=31 + case, base=case * 10 ** 6,
                                 sharing=case % 2))


@pytest.mark.parametrize("app,kw", APPS)
def test_managed_graph(app, kw):
    """Edge arrays in unified memory (--umgraph): same walks."""
    arrs = graphs.ragged()
    starts = np.arange(arrs["n_rows"], dtype=np.int32)
    assert_same(run_both(arrs, app, kw, starts, fw.GROUP_STRIP, managed=True))


def test_host_threads_share_an_engine():
    """Calls on one engine from several host threads are serialised by the library; calls on two
    engines of the same device run side by side.  Every thread gets the single-thread walks."""
    import threading
    g = graphs.config1()
    starts = np.arange(g.V, dtype=np.int32)
    engines = [fw.Engine(g, 0), fw.Engine(g, 0)]
    prms = [fw.make_params(fw.APP_DEEPWALK, d=40, seed=5), fw.make_params(fw.APP_PPR, d=80, tp=0.2, seed=6),
            fw.make_params(fw.APP_NODE2VEC, d=30, p=2.0, q=0.5, seed=7)]
    expect = [engines[0].walk(p, starts)[0] for p in prms]
    got, errors = {}, []

    def work(tid):
        try:
            for rep in range(4):
                k = (tid + rep) % len(prms)
                res, st = engines[tid % 2].walk(prms[k], starts)
                assert st.device_status == 0
                got[(tid, rep)] = (k, res)
        except Exception as exc:  # noqa: BLE001
            errors.append(exc)

    threads = [threading.Thread(target=work, args=(t,)) for t in range(6)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors
    assert len(got) == 24
    for k, res in got.values():
        assert (res == expect[k]).all()
    for e in engines:
        e.close()
    g.close()
