"""The flowwalker command line: the reference's flags (src/main.cu:40-80), its flag rewriting
and result consumers, on top of the C ABI."""
import json
import os
import subprocess

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs
import oracle_lib as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CLI = os.path.join(ROOT, "flowwalker_artifact_b200", "flowwalker")


def run(*args, **kw):
    return subprocess.run([CLI] + list(args), capture_output=True, text=True, timeout=600, **kw)


def test_flag_errors_and_help():
    assert os.path.exists(CLI), "build the CLI with python -m flowwalker_artifact_b200.build"
    r = run("--help")
    assert r.returncode == 0
    for flag in ("--input", "--n", "--all", "--d", "--deepwalk", "--ppr", "--node2vec", "--metapath", "--tp",
                 "--p", "--q", "--schema", "--batchsize", "--autobatch", "--headroom", "--printresult",
                 "--printworkload", "--save_degree", "--b_file", "--walkmode", "--dprs", "--syn", "--lognorm",
                 "--shards"):
        assert flag + " " in r.stdout, flag
    assert run("--bogus").returncode == 2
    assert run("--n", "abc").returncode == 2
    assert run("--n").returncode == 2
    r = run("--input", "/nonexistent/prefix", "--deepwalk")
    assert r.returncode == 1 and "cannot open" in r.stderr


def test_convert_edgelist(tmp_path):
    el = tmp_path / "t.edgelist"
    el.write_text("1 2\n2 3\n3 1\n3 4\n")
    prefix = str(tmp_path / "t")
    r = run("--edgelist", str(el), "--save_csr", prefix)
    assert r.returncode == 0, r.stdout + r.stderr
    g = fw.Graph.load(prefix, True, True)
    assert (g.V, g.E) == (4, 8) and g.adj[:2].tolist() == [1, 2]


def test_needs_exactly_one_app(tmp_path):
    g = graphs.config1()
    prefix = str(tmp_path / "g")
    g.save(prefix)
    r = run("--input", prefix)
    assert r.returncode == 0 and "Please choose a walk mode" in r.stdout


@pytest.mark.gpu
@pytest.mark.parametrize("app,flags,kw", [
    (fw.APP_DEEPWALK, ["--deepwalk", "--d=20"], dict(d=20)),
    (fw.APP_NODE2VEC, ["--node2vec", "--d", "20", "--p=0.5", "--q", "2"], dict(d=20, p=0.5, q=2.0)),
    (fw.APP_METAPATH, ["--metapath", "--schema=1,2,3"], dict(d=3, schema=[1, 2, 3])),
    (fw.APP_PPR, ["--ppr", "--tp=0.1", "--umgraph"], dict(d=80, tp=0.1)),
])
def test_cli_walks_match_the_golden_walker(tmp_path, app, flags, kw):
    g = graphs.config1()
    prefix = str(tmp_path / "g")
    g.save(prefix)
    out = str(tmp_path / "walks.bin")
    bucket = str(tmp_path / "bucket.csv")
    r = run("--input", prefix, "--all", "--printworkload", "--save_degree", "--b_file", bucket,
            "--save_result", out, "--seed=77", *flags)
    assert r.returncode == 0, r.stdout + r.stderr
    walks = np.fromfile(out, dtype=np.int32).reshape(g.V, kw["d"] + 1)
    starts = np.arange(g.V, dtype=np.int32)
    if app == fw.APP_PPR:  # the reference's PPR starts every query at the vertex of largest out-degree
        starts[:] = g.max_degree()[0]
    ref, steps, scanned, _ = O.graph_walk(g, app, starts, seed=77, **kw)
    assert (walks == ref).all()
    assert "Total sampled vertex: %d" % steps in r.stdout
    assert "Total sampled edge: %d" % scanned in r.stdout
    summary = json.loads([ln for ln in r.stdout.splitlines() if ln.startswith("{")][-1])
    assert summary["steps"] == steps and summary["scanned"] == scanned and summary["device_status"] == 0
    rows = [ln.split(",") for ln in open(bucket).read().split()]
    assert sum(int(c) for _, c in rows) == steps


@pytest.mark.gpu
def test_cli_batches_and_printresult(tmp_path):
    g = graphs.config1()
    prefix = str(tmp_path / "g")
    g.save(prefix)
    out = str(tmp_path / "walks.bin")
    r = run("--input", prefix, "--ppr", "--n", "1000", "--uniformstarts", "--startseed=9", "--batch",
            "--batchsize", "300", "--printresult", "--save_result", out)
    assert r.returncode == 0, r.stdout + r.stderr
    walks = np.fromfile(out, dtype=np.int32).reshape(1000, 81)
    ref = O.graph_walk(g, fw.APP_PPR, walks[:, 0].copy(), d=80, tp=0.2)[0]
    assert (walks == ref).all()
    assert r.stdout.count("Walker ") == 100 and "Total length=" in r.stdout
    # reference default for PPR: every query starts at the vertex of largest out-degree
    r = run("--input", prefix, "--ppr", "--n", "50", "--save_result", out)
    assert r.returncode == 0
    assert (np.fromfile(out, dtype=np.int32).reshape(50, 81)[:, 0] == g.max_degree()[0]).all()


@pytest.mark.gpu
def test_cli_two_gpus_and_int64_offsets(tmp_path):
    """Queries sharded over two devices reproduce the single-device table; 64-bit offset files load."""
    import ctypes
    n_dev = ctypes.c_int(0)
    fw.lib().fw_device_count(ctypes.byref(n_dev))
    g = fw.rmat(12, 16 << 12, weight_range=(0.0, 1.0), n_labels=5, xadj_bits=64)
    prefix = str(tmp_path / "g64")
    g.save(prefix)
    out1 = str(tmp_path / "w1.bin")
    r = run("--input", prefix, "--deepwalk", "--all", "--d", "12", "--save_result", out1)
    assert r.returncode == 0, r.stdout + r.stderr
    ref = O.graph_walk(g, fw.APP_DEEPWALK, np.arange(g.V, dtype=np.int32), d=12)[0]
    assert (np.fromfile(out1, dtype=np.int32).reshape(g.V, 13) == ref).all()
    # three shards on one device: the sharded path (id ranges, id bases, one engine and one host
    # thread per shard, results merged) with whatever number of devices is visible
    out3 = str(tmp_path / "w3.bin")
    r = run("--input", prefix, "--deepwalk", "--all", "--d", "12", "--shards", "3", "--save_result", out3)
    assert r.returncode == 0, r.stdout + r.stderr
    assert (np.fromfile(out3, dtype=np.int32).reshape(g.V, 13) == ref).all()
    r = run("--input", prefix, "--deepwalk", "--all", "--d", "12", "--shards", "3", "--interleave",
            "--save_result", out3)
    assert r.returncode == 0, r.stdout + r.stderr
    assert (np.fromfile(out3, dtype=np.int32).reshape(g.V, 13) == ref).all()
    if n_dev.value < 2:
        pytest.skip("one visible device: the two-device half of this test needs two")
    out2 = str(tmp_path / "w2.bin")
    r = run("--input", prefix, "--deepwalk", "--all", "--d", "12", "--gpus", "2", "--save_result", out2)
    assert r.returncode == 0, r.stdout + r.stderr
    assert (np.fromfile(out2, dtype=np.int32).reshape(g.V, 13) == ref).all()


def test_lognormal_weights_are_seeded_and_log_normal():
    """--lognorm's weights (include/graph.cuh:79-91: log-normal, mean 0, sigma 3): a function of the
    seed alone (Philox + Box-Muller, no library distribution object), with the moments asked for."""
    w = fw.lognormal_weights(200001)
    assert w.dtype == np.float32 and (w > 0).all() and np.isfinite(w).all()
    assert [float(x).hex() for x in w[:4]] == ["0x1.3fc2700000000p-2", "0x1.7bd8440000000p-3",
                                               "0x1.8436b20000000p+7", "0x1.4381020000000p+3"]
    assert (fw.lognormal_weights(1001) == w[:1001]).all()          # a prefix, whatever the count
    assert (fw.lognormal_weights(1000, seed=5) != w[:1000]).any()
    lg = np.log(w.astype(np.float64))
    assert abs(lg.mean()) < 0.03 and abs(lg.std() - 3.0) < 0.03
    z = lg / 3.0                                                     # standard normal: check a few quantiles
    for qq, zq in ((0.1, -1.2816), (0.5, 0.0), (0.9, 1.2816), (0.99, 2.3263)):
        assert abs(np.quantile(z, qq) - zq) < 0.03
    small = fw.lognormal_weights(5, mean=1.0, sigma=0.0)
    assert np.allclose(small, np.e, rtol=1e-6)


@pytest.mark.gpu
def test_cli_lognorm_walks_use_those_weights(tmp_path):
    g = graphs.config1()
    prefix = str(tmp_path / "g")
    g.save(prefix)
    out = str(tmp_path / "walks.bin")
    r = run("--input", prefix, "--deepwalk", "--all", "--d", "15", "--lognorm", "--save_result", out)
    assert r.returncode == 0, r.stdout + r.stderr
    walks = np.fromfile(out, dtype=np.int32).reshape(g.V, 16)
    ref = O.walk(g.xadj, g.adj, fw.lognormal_weights(g.E), None, fw.APP_DEEPWALK,
                 np.arange(g.V, dtype=np.int32), d=15)[0]
    assert (walks == ref).all()
