"""The C-ABI library loads, exports what include/flowwalker.h declares, and reads/writes the
reference's on-disk CSR.  No GPU needed (no compute calls)."""
import ctypes
import os
import re

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "flowwalker.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(fw_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = declared_functions()
    assert len(names) >= 15 and "fw_walk" in names and "fw_walk_batch" in names
    L = ctypes.CDLL(fw.lib_path())
    for nm in names:
        assert hasattr(L, nm), "libflowwalker.so does not export " + nm


def test_bench_profile_table_names_the_built_kernels(monkeypatch):
    """bench.py reports DRAM traffic only from an ncu capture of the kernel revision it runs: the
    bench workload's entry has to name the revision the library was built from, or the bench line
    would carry traffic = null."""
    import importlib.util
    spec = importlib.util.spec_from_file_location("fw_bench", os.path.join(ROOT, "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    entry = bench.PROFILED[("deepwalk", 22, 16, 80, 64)]
    assert entry["kernel_revision"] == fw.lib().fw_kernel_revision().decode()
    assert 0 < entry["dram_per_algorithmic_byte"] < 1 and 0 < entry["issue_active"] <= 1
    import sys
    monkeypatch.setattr(sys, "argv", ["bench.py"])
    args = bench.parse()  # the default workload is the one the table's entry is keyed by
    assert (args.app, args.scale, args.edge_factor, args.d, args.group or 64) == ("deepwalk", 22, 16, 80, 64)
    assert (args.gpus, args.steps >= 3, args.warmup >= 3) == (1, True, True)


def test_missing_library_fails_loudly(monkeypatch, tmp_path):
    import flowwalker_artifact_b200._binding as B
    monkeypatch.setattr(B, "_lib", None)
    monkeypatch.setattr(B, "_HERE", str(tmp_path))
    with pytest.raises(fw.FlowWalkerError):
        B.lib()


def test_rmat_properties_and_determinism():
    g = fw.rmat(12, 16 << 12, weight_range=(1.0, 5.0), n_labels=5)
    h = fw.rmat(12, 16 << 12, weight_range=(1.0, 5.0), n_labels=5)
    assert g.E == h.E and (g.adj == h.adj).all() and (g.weight == h.weight).all() and (g.label == h.label).all()
    xa = g.xadj.astype(np.int64)
    assert xa[0] == 0 and xa[-1] == g.E and (np.diff(xa) >= 0).all()
    src = np.repeat(np.arange(g.V), np.diff(xa))
    assert (src != g.adj).all()                                  # no self-loops
    key = src.astype(np.int64) << 32 | g.adj
    assert (np.diff(key) > 0).all()                              # sorted rows, no duplicates
    assert g.weight.min() >= 1.0 and g.weight.max() < 5.0
    assert set(np.unique(g.label)) == {0, 1, 2, 3, 4}
    assert 0.15 < (np.diff(xa) == 0).mean() < 0.7                # directed R-MAT: many dead ends
    other = fw.rmat(12, 16 << 12, seed=2)
    assert other.E != g.E or (other.adj != g.adj).any()
    g64 = fw.rmat(12, 16 << 12, xadj_bits=64)
    assert g64.xadj.dtype == np.int64 and (g64.xadj == xa).all()


def test_config1_shape():
    import graphs
    g = graphs.config1()
    assert (g.V, g.E) == (7115, 103689)
    assert g.adj.max() < 7115


def test_save_load_roundtrip_32_and_64(tmp_path):
    for bits in (32, 64):
        g = fw.rmat(10, 8 << 10, weight_range=(0.0, 1.0), n_labels=5, xadj_bits=bits)
        prefix = str(tmp_path / ("g%d" % bits))
        g.save(prefix)
        assert os.path.getsize(prefix + "_xadj.bin") == 8 + (bits // 8) * (g.V + 1)
        hdr = np.fromfile(prefix + "_xadj.bin", dtype=np.uint32, count=2)
        assert hdr.tolist() == [g.V, g.E]
        for need_w, need_l in ((True, False), (False, True), (True, True)):
            h = fw.Graph.load(prefix, need_w, need_l)
            assert (h.V, h.E, h.xadj_bits) == (g.V, g.E, bits)
            assert (h.xadj == g.xadj).all() and (h.adj == g.adj).all()
            assert (h.weight is not None) == need_w and (h.label is not None) == need_l
            if need_w:
                assert (h.weight == g.weight).all()
            if need_l:
                assert (h.label == g.label).all()


def test_load_errors(tmp_path):
    g = fw.rmat(8, 2000, weight_range=(0.0, 1.0))
    prefix = str(tmp_path / "g")
    g.save(prefix)
    with pytest.raises(fw.FlowWalkerError) as ei:
        fw.Graph.load(str(tmp_path / "nope"))
    assert ei.value.code == -2
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.load(prefix, need_weight=False, need_label=True)   # no label file written
    with open(prefix + "_weight.bin", "ab") as f:
        f.write(b"\0\0\0\0")
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.load(prefix)                                       # weight file of the wrong size
    raw = bytearray(open(prefix + "_xadj.bin", "rb").read())
    with open(prefix + "_xadj.bin", "wb") as f:
        f.write(raw[:-2])
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.load(prefix, need_weight=False)                    # truncated offsets
    raw[8 + 4 * 5: 8 + 4 * 6] = (10 ** 9).to_bytes(4, "little")
    with open(prefix + "_xadj.bin", "wb") as f:
        f.write(raw)
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.load(prefix, need_weight=False)                    # offsets not monotone


def test_from_arrays_validation():
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.from_arrays(np.array([0, 2, 1], dtype=np.uint32), np.array([1, 0], dtype=np.int32))
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.from_arrays(np.array([0, 1, 3], dtype=np.uint32), np.array([1, 0], dtype=np.int32))
    g = fw.Graph.from_arrays(np.array([0, 1, 2], dtype=np.int64), np.array([1, 0], dtype=np.int32),
                             weight=np.array([1.0, 2.0], dtype=np.float32))
    assert g.xadj_bits == 64 and g.max_degree() == (0, 1)


# the reference checkout, when one is at hand (FW_REFERENCE_DIR, as oracle/build_ref.sh reads it)
REFERENCE_SAMPLE = os.path.join(os.environ.get("FW_REFERENCE_DIR", ""), "data", "wiki-Vote")


@pytest.mark.skipif(not os.path.exists(REFERENCE_SAMPLE + "_xadj.bin"),
                    reason="FW_REFERENCE_DIR does not point at a reference checkout with its sample graph")
def test_reads_the_reference_sample_graph():
    g = fw.Graph.load(REFERENCE_SAMPLE, True, True)
    assert (g.V, g.E) == (7115, 201524)
    assert g.max_degree()[1] == 1065
    assert g.weight.min() > 0 and g.weight.max() < 5 and set(np.unique(g.label)) == {0, 1, 2, 3, 4}


def test_edgelist_converter(tmp_path):
    path = tmp_path / "toy.edgelist"
    path.write_text("# a comment\n10 20\n20 10\n10 30\n30 30\n40 20\n% another\n20 40\n50 10\n")
    g = fw.Graph.from_edgelist(str(path), n_labels=5, weight_range=(1.0, 5.0), seed=3)
    # first appearance: 10->0, 20->1, 30->2, 40->3, 50->4; undirected edges {0-1, 0-2, 1-3, 0-4}
    assert (g.V, g.E) == (5, 8)
    xa = g.xadj.astype(np.int64)
    rows = [g.adj[xa[v]:xa[v + 1]].tolist() for v in range(g.V)]
    assert rows == [[1, 2, 4], [0, 3], [0], [1], [0]]
    w = {(v, int(x)): float(g.weight[e]) for v in range(g.V) for e, x in zip(range(xa[v], xa[v + 1]), g.adj[xa[v]:xa[v + 1]])}
    lab = {(v, int(x)): int(g.label[e]) for v in range(g.V) for e, x in zip(range(xa[v], xa[v + 1]), g.adj[xa[v]:xa[v + 1]])}
    for (u, v), val in w.items():
        assert w[(v, u)] == val and 1.0 <= val < 5.0 and lab[(v, u)] == lab[(u, v)] and 0 <= lab[(u, v)] < 5
    again = fw.Graph.from_edgelist(str(path), n_labels=5, weight_range=(1.0, 5.0), seed=3)
    assert (again.weight == g.weight).all() and (again.label == g.label).all()
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.from_edgelist(str(tmp_path / "missing.edgelist"))
    bad = tmp_path / "bad.edgelist"
    bad.write_text("1 2\nhello\n")
    with pytest.raises(fw.FlowWalkerError):
        fw.Graph.from_edgelist(str(bad))
