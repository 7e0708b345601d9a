"""fw_walk_csr_noalloc: the entry point for callers that cannot allocate device memory
at call time (a plugin inside another framework's memory pool, a serving loop that must
not pay cudaMalloc's device-wide synchronisation, a process with a frozen allocator).
Its scratch is a fixed array inside the loaded module, so its walks must equal those of
fw_walk_device, which uses scratch allocated by the engine, and those of the CPU golden
walker -- on the first call, which also does the one-time address lookup, and on later
calls, which find the previous call's counters in the array.

The file name sorts last so that a run that stops at the first failure has already run
every other test; nothing here depends on what ran before (the entry point's first call in
a process does its own set-up), and the file passes alone in a fresh process as well."""
import ctypes

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs
import oracle_lib as O

pytestmark = pytest.mark.gpu


class _DeviceCsr:
    """The config-1 graph as raw device arrays the way a caller of this entry point holds them:
    offsets of the width asked for, edge arrays readable for whole 16-byte quads past E."""

    def __init__(self, g, bits):
        import torch
        self.torch = torch
        self.dev = torch.device("cuda", 0)
        self.g, self.bits = g, bits
        self.xadj_host = g.xadj.astype(np.int64 if bits == 64 else np.uint32)
        view = self.xadj_host.view(np.int64 if bits == 64 else np.int32)  # torch has no uint32 tensors
        self.xadj = torch.from_numpy(view.copy()).to(self.dev)
        self.adj, self.w, self.lab = (self._padded(a) for a in (g.adj, g.weight, g.label))

    def _padded(self, a):
        torch = self.torch
        t = torch.zeros(len(a) + 8, dtype=torch.from_numpy(a[:1].copy()).dtype, device=self.dev)
        t[:len(a)] = torch.from_numpy(a.copy()).to(self.dev)
        return t

    def call(self, prm, starts_dev, n, out_dev, stats=None, hist=None, weight=True, label=True):
        return fw.lib().fw_walk_csr_noalloc(
            0, self.g.V, self.g.E, self.xadj.data_ptr(), self.bits, self.adj.data_ptr(),
            self.w.data_ptr() if weight else None, self.lab.data_ptr() if label else None,
            ctypes.byref(prm[0]), starts_dev.data_ptr(), n, out_dev.data_ptr(), None,
            None if stats is None else ctypes.byref(stats), None if hist is None else hist.ctypes.data)

    def oracle(self, app, starts, **kw):
        g = self.g
        return O.walk(self.xadj_host, g.adj, g.weight, g.label, app, starts, **kw)


CALLS = [
    (fw.APP_DEEPWALK, dict(d=80)),
    (fw.APP_PPR, dict(d=80, tp=0.2)),
    (fw.APP_METAPATH, dict(d=80, schema=[0, 1, 2, 3, 4])),
    (fw.APP_NODE2VEC, dict(d=40, p=0.5, q=2.0)),
    (fw.APP_NODE2VEC, dict(d=12, p=2.0, q=0.5, group_mode=fw.GROUP_EDGE)),
]


@pytest.mark.parametrize("bits", [64, 32])
def test_noalloc_matches_engine_and_oracle_call_after_call(bits):
    """Five calls in a row on the shared scratch array (each finds the previous one's counters
    there): the walks, the counters and the length histogram equal fw_walk_device's and the CPU
    golden walker's, bit for bit, for both offset widths, node2vec included."""
    import torch
    L = fw.lib()
    g = graphs.config1()
    eng = fw.Engine(g, 0)
    csr = _DeviceCsr(g, bits)
    torch.cuda.synchronize()
    for call, (app, kw) in enumerate(CALLS):
        n = 3000 + 500 * call
        d = kw["d"]
        starts_host = graphs.config1_starts(n, seed=40 + call)
        starts = torch.from_numpy(starts_host).to(csr.dev)
        prm = fw.make_params(app, seed=7 + call, query_id_base=1000 * call, **kw)
        want = torch.empty((n, d + 1), dtype=torch.int32, device=csr.dev)
        hist_want = np.zeros(d + 1, dtype=np.uint64)
        st_want = eng.walk_device(prm, starts.data_ptr(), n, want.data_ptr(), hist=hist_want)
        got = torch.full((n, d + 1), -7, dtype=torch.int32, device=csr.dev)
        torch.cuda.synchronize()
        hist_got = np.zeros(d + 1, dtype=np.uint64)
        st = fw.WalkStats()
        assert csr.call(prm, starts, n, got, st, hist_got) == 0, L.fw_last_error()
        assert torch.equal(got, want)  # integer walks: bit-exact, as in the other parity tests
        assert (st.steps, st.scanned, st.device_status) == (st_want.steps, st_want.scanned, 0)
        assert (hist_got == hist_want).all()
        okw = {k: v for k, v in kw.items() if k != "group_mode"}
        ref, steps, scanned, rhist = csr.oracle(app, starts_host, seed=7 + call, query_id_base=1000 * call,
                                                group_mode=kw.get("group_mode", 64), **okw)
        assert (got.cpu().numpy() == ref).all()
        assert (st.steps, st.scanned) == (steps, scanned) and (hist_got == rhist).all()
    eng.close()


def test_noalloc_limits_and_no_device_allocation():
    """The documented limits: d = 4095 and a 64-entry schema are served; d beyond the fixed
    scratch is refused, not truncated; stats and len_hist may be NULL; and the amount of free
    device memory is the same before and after a call (after the set-up call)."""
    import torch
    L = fw.lib()
    g = graphs.config1()
    csr = _DeviceCsr(g, 32)
    n = 512
    starts_host = graphs.config1_starts(n, seed=77)
    starts = torch.from_numpy(starts_host).to(csr.dev)
    # largest d: the histogram fills the whole scratch array and the largest shared-memory block
    for app, kw in ((fw.APP_DEEPWALK, dict(d=4095)), (fw.APP_NODE2VEC, dict(d=4095, p=2.0, q=0.5))):
        prm = fw.make_params(app, seed=3, **kw)
        got = torch.full((n, 4096), -7, dtype=torch.int32, device=csr.dev)
        st = fw.WalkStats()
        hist = np.zeros(4096, dtype=np.uint64)
        assert csr.call(prm, starts, n, got, st, hist) == 0, L.fw_last_error()
        ref, steps, scanned, rhist = csr.oracle(app, starts_host, seed=3, **kw)
        assert (got.cpu().numpy() == ref).all() and (st.steps, st.scanned) == (steps, scanned)
        assert (hist == rhist).all()
    # longest schema, labels only (weights NULL), no stats, no histogram
    schema = (np.arange(64) * 3 % 5).astype(np.int32)
    prm = fw.make_params(fw.APP_METAPATH, d=64, schema=schema, seed=4)
    got = torch.full((n, 65), -7, dtype=torch.int32, device=csr.dev)
    assert csr.call(prm, starts, n, got, None, None, weight=False) == 0, L.fw_last_error()
    ref, _, _, _ = csr.oracle(fw.APP_METAPATH, starts_host, d=64, schema=schema, seed=4)
    assert (got.cpu().numpy() == ref).all()
    # a second, identical call: same walks, and no device memory taken or given back
    torch.cuda.synchronize()
    free_before, _ = torch.cuda.mem_get_info(0)
    again = torch.full((n, 65), -7, dtype=torch.int32, device=csr.dev)  # torch's allocation, outside the bracket
    torch.cuda.synchronize()
    free_mid, _ = torch.cuda.mem_get_info(0)
    assert csr.call(prm, starts, n, again, None, None, weight=False) == 0, L.fw_last_error()
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info(0)
    assert free_after == free_mid <= free_before
    assert torch.equal(again, got)
    # sizes beyond the fixed scratch are refused, not truncated
    prm = fw.make_params(fw.APP_DEEPWALK, d=4096)
    assert csr.call(prm, starts, 1, got, None, None, label=False) == -1
    assert b"exceeds the fixed scratch" in L.fw_last_error()
    # a device that is not there is refused before anything is looked up
    prm = fw.make_params(fw.APP_DEEPWALK, d=8)
    rc = L.fw_walk_csr_noalloc(63, g.V, g.E, csr.xadj.data_ptr(), 32, csr.adj.data_ptr(), csr.w.data_ptr(), None,
                               ctypes.byref(prm[0]), starts.data_ptr(), 1, got.data_ptr(), None, None, None)
    assert rc != 0 and b"out of range" in L.fw_last_error()
