import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))

APP_DEEPWALK, APP_PPR, APP_NODE2VEC, APP_METAPATH = 0, 1, 2, 3
GROUP_EDGE, GROUP_STRIP = 1, 64
ENGINE_MANAGED = 4


class FlowWalkerError(RuntimeError):
    def __init__(self, code, message):
        super().__init__("flowwalker error %d: %s" % (code, message))
        self.code = code


class _Params(ctypes.Structure):
    _fields_ = [("app", ctypes.c_int32), ("d", ctypes.c_int32), ("tp", ctypes.c_double),
                ("p", ctypes.c_double), ("q", ctypes.c_double),
                ("schema", ctypes.POINTER(ctypes.c_int32)), ("schema_len", ctypes.c_int32),
                ("group_mode", ctypes.c_int32), ("seed", ctypes.c_uint64),
                ("query_id_base", ctypes.c_uint64), ("query_id_stride", ctypes.c_uint64)]


class WalkStats(ctypes.Structure):
    _fields_ = [("steps", ctypes.c_uint64), ("scanned", ctypes.c_uint64),
                ("device_ms", ctypes.c_double), ("total_ms", ctypes.c_double),
                ("device_status", ctypes.c_uint32), ("launches", ctypes.c_uint32)]


class _Rmat(ctypes.Structure):
    _fields_ = [("scale", ctypes.c_int32), ("xadj_bits", ctypes.c_int32), ("draws", ctypes.c_int64),
                ("a", ctypes.c_double), ("b", ctypes.c_double), ("c", ctypes.c_double),
                ("seed", ctypes.c_uint64), ("v_limit", ctypes.c_int64), ("e_target", ctypes.c_int64),
                ("weight_lo", ctypes.c_float), ("weight_hi", ctypes.c_float),
                ("weight_seed", ctypes.c_uint64), ("n_labels", ctypes.c_int32),
                ("label_seed", ctypes.c_uint64), ("device", ctypes.c_int32)]


_lib = None


def lib_path():
    """Path of the shared library; FLOWWALKER_LIB overrides the in-tree build."""
    return os.environ.get("FLOWWALKER_LIB") or os.path.join(_HERE, "libflowwalker.so")


def lib():
    """Loads libflowwalker.so; raises when it has not been built (no fallback exists)."""
    global _lib
    if _lib is None:
        path = lib_path()
        if not os.path.exists(path):
            raise FlowWalkerError(-100, "%s is missing: run `python -m flowwalker_artifact_b200.build`" % path)
        L = ctypes.CDLL(path)
        L.fw_last_error.restype = ctypes.c_char_p
        L.fw_kernel_revision.restype = ctypes.c_char_p
        vp, i64, i32 = ctypes.c_void_p, ctypes.c_int64, ctypes.c_int32
        L.fw_device_count.argtypes = [ctypes.POINTER(ctypes.c_int)]
        L.fw_graph_load.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(vp)]
        L.fw_graph_save.argtypes = [vp, ctypes.c_char_p]
        L.fw_graph_from_arrays.argtypes = [i64, i64, vp, ctypes.c_int, vp, vp, vp, ctypes.POINTER(vp)]
        L.fw_graph_from_edgelist.argtypes = [ctypes.c_char_p, i32, ctypes.c_float, ctypes.c_float,
                                             ctypes.c_uint64, ctypes.POINTER(vp)]
        L.fw_rmat_generate.argtypes = [ctypes.POINTER(_Rmat), ctypes.POINTER(vp)]
        L.fw_lognormal_weights.argtypes = [i64, ctypes.c_double, ctypes.c_double, ctypes.c_uint64, vp]
        L.fw_graph_info.argtypes = [vp, ctypes.POINTER(i64), ctypes.POINTER(i64), ctypes.POINTER(i32),
                                    ctypes.POINTER(i32), ctypes.POINTER(i32)]
        L.fw_graph_arrays.argtypes = [vp] + [ctypes.POINTER(vp)] * 4
        L.fw_graph_max_degree.argtypes = [vp, ctypes.POINTER(i64), ctypes.POINTER(i64)]
        L.fw_graph_destroy.argtypes = [vp]
        L.fw_graph_destroy.restype = None
        L.fw_engine_create.argtypes = [vp, ctypes.c_int, ctypes.c_int, ctypes.POINTER(vp)]
        L.fw_engine_destroy.argtypes = [vp]
        L.fw_engine_destroy.restype = None
        L.fw_engine_device.argtypes = [vp, ctypes.POINTER(ctypes.c_int), ctypes.POINTER(ctypes.c_int)]
        L.fw_engine_set_sharing.argtypes = [vp, ctypes.c_int]
        L.fw_engine_set_hub_batching.argtypes = [vp, ctypes.c_int]
        L.fw_engine_set_early_delivery.argtypes = [vp, ctypes.c_int]
        L.fw_engine_hubs.argtypes = [vp, ctypes.c_int, ctypes.POINTER(i32), ctypes.POINTER(ctypes.c_uint32)]
        L.fw_walk_device.argtypes = [vp, ctypes.POINTER(_Params), vp, i64, vp, vp,
                                     ctypes.POINTER(WalkStats), vp]
        L.fw_walk.argtypes = [vp, ctypes.POINTER(_Params), vp, i64, vp, ctypes.POINTER(WalkStats), vp]
        L.fw_walk_batch.argtypes = [vp, ctypes.POINTER(_Params), vp, i64, i64, i32,
                                    ctypes.POINTER(vp), ctypes.POINTER(WalkStats), vp]
        L.fw_walk_batch_into.argtypes = [vp, ctypes.POINTER(_Params), vp, i64, i64, i32, vp,
                                         ctypes.POINTER(WalkStats), vp]
        L.fw_free_pinned.argtypes = [vp]
        L.fw_free_pinned.restype = None
        L.fw_selftest_wait_timeout.argtypes = [ctypes.c_int, ctypes.c_uint32, ctypes.POINTER(ctypes.c_uint32)]
        L.fw_walk_csr_noalloc.argtypes = [ctypes.c_int, i64, i64, vp, ctypes.c_int, vp, vp, vp,
                                          ctypes.POINTER(_Params), vp, i64, vp, vp,
                                          ctypes.POINTER(WalkStats), vp]
        _lib = L
    return _lib


def _check(rc):
    if rc != 0:
        raise FlowWalkerError(rc, lib().fw_last_error().decode("utf-8", "replace"))


def make_params(app, d=80, tp=0.2, p=2.0, q=0.5, schema=None, group_mode=0, seed=1337, query_id_base=0,
                query_id_stride=1):
    """Returns (struct, keepalive) for a fw_walk_params."""
    prm = _Params()
    prm.app, prm.d, prm.tp, prm.p, prm.q = app, d, tp, p, q
    keep = None
    if schema is not None:
        keep = np.ascontiguousarray(schema, dtype=np.int32)
        prm.schema = keep.ctypes.data_as(ctypes.POINTER(ctypes.c_int32))
        prm.schema_len = len(keep)
    prm.group_mode, prm.seed, prm.query_id_base = group_mode, seed, query_id_base
    prm.query_id_stride = query_id_stride
    return prm, keep


class Graph:
    """Host CSR (fw_graph)."""

    def __init__(self, handle):
        self._h = ctypes.c_void_p(handle)
        V, E = ctypes.c_int64(), ctypes.c_int64()
        bits, hw, hl = ctypes.c_int32(), ctypes.c_int32(), ctypes.c_int32()
        _check(lib().fw_graph_info(self._h, V, E, bits, hw, hl))
        self.V, self.E, self.xadj_bits = V.value, E.value, bits.value
        ptrs = [ctypes.c_void_p() for _ in range(4)]
        _check(lib().fw_graph_arrays(self._h, *ptrs))

        def view(ptr, n, dtype):
            if not ptr.value:
                return None
            if n == 0:
                return np.zeros(0, dtype=dtype)
            buf = (ctypes.c_char * (n * np.dtype(dtype).itemsize)).from_address(ptr.value)
            return np.frombuffer(buf, dtype=dtype)

        self.xadj = view(ptrs[0], self.V + 1, np.int64 if self.xadj_bits == 64 else np.uint32)
        self.adj = view(ptrs[1], self.E, np.int32)
        self.weight = view(ptrs[2], self.E, np.float32) if hw.value else None
        self.label = view(ptrs[3], self.E, np.int32) if hl.value else None

    @classmethod
    def load(cls, prefix, need_weight=True, need_label=False):
        h = ctypes.c_void_p()
        _check(lib().fw_graph_load(os.fsencode(prefix), int(need_weight), int(need_label), h))
        return cls(h.value)

    @classmethod
    def from_edgelist(cls, path, n_labels=5, weight_range=(1.0, 5.0), seed=1):
        h = ctypes.c_void_p()
        _check(lib().fw_graph_from_edgelist(os.fsencode(path), n_labels, weight_range[0], weight_range[1], seed, h))
        return cls(h.value)

    @classmethod
    def from_arrays(cls, xadj, adj, weight=None, label=None):
        xadj = np.ascontiguousarray(xadj)
        if xadj.dtype not in (np.dtype(np.uint32), np.dtype(np.int64)):
            raise TypeError("xadj must be uint32 or int64")
        adj = np.ascontiguousarray(adj, dtype=np.int32)
        w = None if weight is None else np.ascontiguousarray(weight, dtype=np.float32)
        lb = None if label is None else np.ascontiguousarray(label, dtype=np.int32)
        h = ctypes.c_void_p()
        _check(lib().fw_graph_from_arrays(len(xadj) - 1, len(adj), xadj.ctypes.data,
                                          64 if xadj.dtype == np.int64 else 32, adj.ctypes.data,
                                          None if w is None else w.ctypes.data,
                                          None if lb is None else lb.ctypes.data, h))
        return cls(h.value)

    def save(self, prefix):
        _check(lib().fw_graph_save(self._h, os.fsencode(prefix)))

    def max_degree(self):
        v, dg = ctypes.c_int64(), ctypes.c_int64()
        _check(lib().fw_graph_max_degree(self._h, v, dg))
        return v.value, dg.value

    def close(self):
        if self._h:
            self.xadj = self.adj = self.weight = self.label = None
            lib().fw_graph_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def rmat(scale, draws, a=0.57, b=0.19, c=0.19, seed=1, v_limit=0, e_target=0, weight_range=(0.0, 1.0),
         weight_seed=2, n_labels=0, label_seed=3, xadj_bits=32, device=-1):
    """Seeded R-MAT graph (fw_rmat_generate); device=-1 generates on the host."""
    r = _Rmat()
    r.scale, r.xadj_bits, r.draws = scale, xadj_bits, draws
    r.a, r.b, r.c, r.seed = a, b, c, seed
    r.v_limit, r.e_target = v_limit, e_target
    r.weight_lo, r.weight_hi = (weight_range if weight_range else (0.0, 0.0))
    r.weight_seed, r.n_labels, r.label_seed, r.device = weight_seed, n_labels, label_seed, device
    h = ctypes.c_void_p()
    _check(lib().fw_rmat_generate(r, h))
    return Graph(h.value)


class Engine:
    """Device replica of a graph on one GPU (fw_engine)."""

    def __init__(self, graph, device=0, which=0, managed=False):
        self._h = ctypes.c_void_p()
        _check(lib().fw_engine_create(graph._h, device, which | (ENGINE_MANAGED if managed else 0), self._h))
        dev, sms = ctypes.c_int(), ctypes.c_int()
        _check(lib().fw_engine_device(self._h, dev, sms))
        self.device, self.sm_count = dev.value, sms.value

    def set_sharing(self, mode):
        """-1: by max degree (default), 0: never, 1: always share very long rows between warps."""
        _check(lib().fw_engine_set_sharing(self._h, mode))

    def set_hub_batching(self, mode):
        """-1: when the graph has hub vertices and the call is large enough (default), 0: never,
        1: whenever the graph has hubs, 2: as 1 and batching to the last walker.  Walkers that meet
        at a hub share one sweep of its row."""
        _check(lib().fw_engine_set_hub_batching(self._h, mode))

    def set_early_delivery(self, mode):
        """-1 (default): a hub-batched call whose result buffer is page-locked host memory writes
        the rows of ended walks to it while the others walk on, where the walk is long enough for
        that to pay; 0: one copy after the last launch; 1: always deliver; 2: deliver, then fall
        back to the copy (1 and 2 are for tests)."""
        _check(lib().fw_engine_set_early_delivery(self._h, mode))

    def hubs(self, which=0):
        """(number of hub vertices, row length from which a vertex is a hub) for the limit of
        1,016 neighbours (which=0) or of 504 (which=1)."""
        n, t = ctypes.c_int32(), ctypes.c_uint32()
        _check(lib().fw_engine_hubs(self._h, which, n, t))
        return n.value, t.value

    def walk(self, params, starts, want_hist=False):
        """Host buffers in, host result out (fw_walk)."""
        prm, _keep = params
        starts = np.ascontiguousarray(starts, dtype=np.int32)
        n = len(starts)
        out = np.empty((n, prm.d + 1), dtype=np.int32)
        st = WalkStats()
        hist = np.zeros(prm.d + 1, dtype=np.uint64) if want_hist else None
        _check(lib().fw_walk(self._h, prm, starts.ctypes.data, n, out.ctypes.data, st,
                             None if hist is None else hist.ctypes.data))
        return (out, st, hist) if want_hist else (out, st)

    def walk_device(self, params, starts_ptr, n, result_ptr, stream=None, hist=None):
        """Device pointers in and out (fw_walk_device); returns WalkStats."""
        prm, _keep = params
        st = WalkStats()
        _check(lib().fw_walk_device(self._h, prm, starts_ptr, n, result_ptr, stream, st,
                                    None if hist is None else hist.ctypes.data))
        return st

    def walk_batch(self, params, starts, batch_size=0, headroom_mb=512):
        """Double-buffered batches into callee-allocated pinned memory (fw_walk_batch)."""
        prm, _keep = params
        starts = np.ascontiguousarray(starts, dtype=np.int32)
        n = len(starts)
        ptr = ctypes.c_void_p()
        st = WalkStats()
        _check(lib().fw_walk_batch(self._h, prm, starts.ctypes.data, n, batch_size, headroom_mb,
                                   ptr, st, None))
        try:
            cells = n * (prm.d + 1)
            if cells:
                buf = (ctypes.c_int32 * cells).from_address(ptr.value)
                out = np.frombuffer(buf, dtype=np.int32).reshape(n, prm.d + 1).copy()
            else:
                out = np.zeros((0, prm.d + 1), dtype=np.int32)
        finally:
            lib().fw_free_pinned(ptr)
        return out, st

    def close(self):
        if self._h:
            lib().fw_engine_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass


def lognormal_weights(n, mean=0.0, sigma=3.0, seed=1234):
    """Seeded log-normal weights (fw_lognormal_weights): what the CLI's --lognorm puts on the edges."""
    out = np.empty(n, dtype=np.float32)
    _check(lib().fw_lognormal_weights(n, mean, sigma, seed, out.ctypes.data))
    return out
