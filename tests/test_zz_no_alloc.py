"""fw_walk_csr_noalloc: the entry point for callers that cannot allocate device memory
at call time (a plugin inside another framework's memory pool, a serving loop that must
not pay cudaMalloc's device-wide synchronisation, a process with a frozen allocator).
Its scratch is a fixed array inside the loaded module, so its walks must equal those of
fw_walk_device, which uses scratch allocated by the engine -- on the first call, which
also does the one-time address lookup, and on a second call, which finds the previous
call's counters in the array.  Collected last on purpose."""
import ctypes

import numpy as np
import pytest

import flowwalker_artifact_b200 as fw
import graphs

pytestmark = pytest.mark.gpu


def _bind():
    L = fw.lib()
    vp, i64 = ctypes.c_void_p, ctypes.c_int64
    L.fw_walk_csr_noalloc.argtypes = [ctypes.c_int, i64, i64, vp, ctypes.c_int, vp, vp, vp, vp, vp, i64,
                                      vp, vp, ctypes.POINTER(fw.WalkStats), vp]
    return L


def test_noalloc_matches_engine_twice_in_a_row():
    import torch
    L = _bind()
    g = graphs.config1()
    eng = fw.Engine(g, 0)
    dev = torch.device("cuda", 0)

    def padded(a):  # whole 16-byte quads past E stay readable
        t = torch.zeros(len(a) + 8, dtype=torch.from_numpy(a[:1].copy()).dtype, device=dev)
        t[:len(a)] = torch.from_numpy(a.copy()).to(dev)
        return t

    xadj = torch.from_numpy(g.xadj.astype(np.int64)).to(dev)  # 64-bit offsets on this path
    adj, w, lab = padded(g.adj), padded(g.weight), padded(g.label)
    d = 80
    torch.cuda.synchronize()
    for call, (app, kw) in enumerate([(fw.APP_DEEPWALK, {}), (fw.APP_PPR, dict(tp=0.2)),
                                      (fw.APP_METAPATH, dict(schema=[0, 1, 2, 3, 4]))]):
        n = 3000 + 500 * call
        starts = torch.from_numpy(graphs.config1_starts(n, seed=40 + call)).to(dev)
        prm = fw.make_params(app, d=d, seed=7 + call, **kw)
        want = torch.empty((n, d + 1), dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        hist_want = np.zeros(d + 1, dtype=np.uint64)
        st_want = eng.walk_device(prm, starts.data_ptr(), n, want.data_ptr(), hist=hist_want)
        got = torch.full((n, d + 1), -7, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        hist_got = np.zeros(d + 1, dtype=np.uint64)
        st = fw.WalkStats()
        rc = L.fw_walk_csr_noalloc(0, g.V, g.E, xadj.data_ptr(), 64, adj.data_ptr(), w.data_ptr(),
                                   lab.data_ptr(), ctypes.byref(prm[0]), starts.data_ptr(), n,
                                   got.data_ptr(), None, ctypes.byref(st), hist_got.ctypes.data)
        assert rc == 0, L.fw_last_error()
        assert torch.equal(got, want)  # integer walks: bit-exact, as in the other parity tests
        assert (st.steps, st.scanned, st.device_status) == (st_want.steps, st_want.scanned, 0)
        assert (hist_got == hist_want).all()
    # sizes beyond the fixed scratch are refused, not truncated
    prm = fw.make_params(fw.APP_DEEPWALK, d=5000)
    rc = L.fw_walk_csr_noalloc(0, g.V, g.E, xadj.data_ptr(), 64, adj.data_ptr(), w.data_ptr(), None,
                               ctypes.byref(prm[0]), starts.data_ptr(), 1, got.data_ptr(), None, None, None)
    assert rc == -1 and b"exceeds the fixed scratch" in L.fw_last_error()
    eng.close()
