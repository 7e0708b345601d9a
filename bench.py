#!/usr/bin/env python
"""Walk-throughput bench: DeepWalk, all-vertex queries, walk length 80, weighted,
on a seeded synthetic R-MAT scale-22 graph (edge factor 16), one engine per GPU.

A "step" of this bench is one full pass of the hot path: every vertex starts
one walk (n = V queries, up to 80 walk steps each).  With N GPUs the graph is
replicated and every rank walks all V start vertices under its own query-id
range (walk round r of a walks-per-vertex = N job), so per-GPU work is fixed
("weak" scaling) and no collective touches the walk; torch.distributed only
carries the barrier and the final reduction of counters and times.

Prints ONE JSON line (rank 0).  `value` is walk steps per second with inputs
resident in HBM; `e2e` is the same through fw_walk_batch_into with pinned host buffers
(start vertices copied in, the whole walk table copied out).  A pass of this workload is a
hub-batched call: a series of kernel launches in which walkers that meet at a hub vertex share
one sweep of its row, so the walk of a pass is best done in one piece (measured 85.6 / 92.8 /
101.6 / 110.9 ms per end-to-end pass as 1 / 2 / 3 / 4 double-buffered batches: every batch
pays the fixed cost of its own series) and `--e2e-batches` defaults to 1.

With N > 1 the line also carries `strong`: ONE job partitioned over the ranks, the way a
user shards queries over the GPUs of a box -- rank r of R takes the contiguous id range
[r n / R, (r+1) n / R) of the same n queries (and, beside it, the interleaved assignment
id = r mod R) -- for n = V (a short launch per rank: fixed launch and claim cost, tail of the
persistent kernel) and n = R V (as much work per rank as a full pass), each with the time of
every rank, the imbalance max / mean and the efficiency against one GPU; after the timing every
rank checks 256 of its rows against the CPU golden walker (`parity_sample`).
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

APPS = {"deepwalk": 0, "ppr": 1, "node2vec": 2, "metapath": 3}


def parse():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=5)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--app", default="deepwalk", choices=list(APPS))
    ap.add_argument("--scale", type=int, default=22)
    ap.add_argument("--edge-factor", type=int, default=16)
    ap.add_argument("--d", type=int, default=80)
    ap.add_argument("--group", type=int, default=0, help="sampler granularity: 0 default, 1 or 64")
    ap.add_argument("--queries", type=int, default=0, help="0 = all vertices; otherwise seeded uniform starts")
    ap.add_argument("--rmat-a", type=float, default=0.57, help="R-MAT a (b = c = 0.19)")
    ap.add_argument("--weights", default="0,1", help="weights uniform in [lo,hi)")
    ap.add_argument("--xadj-bits", type=int, default=32, choices=[32, 64])
    ap.add_argument("--sharing", type=int, default=-1, choices=[-1, 0, 1],
                    help="warps share very long rows: -1 by the graph's largest degree, 0 never, 1 always")
    ap.add_argument("--hub-batching", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="walkers that meet at a hub share a sweep: -1 when the call is large enough, 0 never, 1 always")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-strong", action="store_true", help="skip the partitioned-job legs of a multi-GPU run")
    ap.add_argument("--no-numa", action="store_true", help="leave the rank's CPU affinity as it is")
    ap.add_argument("--early-delivery", type=int, default=-1, choices=[-1, 0, 1, 2],
                    help="end-to-end leg: -1 rows of ended walks go to the host table while the others walk on where "
                         "the walk is long enough (fw_engine_set_early_delivery), 0 one copy of the table after the "
                         "last launch, 1 always deliver, 2 deliver then fall back to the copy")
    ap.add_argument("--e2e-batches", type=int, default=1, help="double-buffered batches of the end-to-end leg")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.FIELDS,
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons)}


# Counters of the walk that only a profiler sees, per workload (app, scale, edge factor, d, group
# mode): DRAM bytes per algorithmic byte (dram__bytes_read.sum + dram__bytes_write.sum over every
# walk and hub kernel launch of an `ncu` capture of the same call with fewer queries on the same
# graph, over that call's algorithmic bytes; both grow in proportion with the number of queries as
# long as the call uses the same hub limit), the share of issue slots in use and the L2 hit rate
# (time-weighted over the launches).  Each entry names the kernel revision (fw_kernel_revision) it
# was captured on; a line measured on another revision, or on a workload without an entry, reports
# traffic = null with the reason.
PROFILED = {
    ("deepwalk", 22, 16, 80, 64): {
        "kernel_revision": "hub-batched-3",
        "captured_on": "2,700,000-query call on the same graph (profiles/hub_batched_pass_deepwalk_scale22.md)",
        "dram_per_algorithmic_byte": 0.0606, "issue_active": 0.626, "l2_hit_rate": 0.476,
        "instructions_per_step": 317.9,
    },
}


def algorithmic_bytes(app, scanned, steps, n, xadj_bits, prev_scanned=0, as_built=False):
    """Bytes the path has to touch at least once.  Weights (or labels) read once per scanned
    neighbour, plus per step the chosen neighbour id, the two row bounds of the new vertex and the
    result cell, plus per query the start vertex, its row bounds and the first result cell.
    node2vec, as the scope table counts it: weight and neighbour id of every candidate (8 B) and
    one streaming pass over the previous vertex's row per step (4 B per entry, `prev_scanned`).
    `as_built`: what this engine's node2vec needs as a minimum instead -- its sweep reads the
    weights only (4 B per candidate) and looks at neighbour ids for the few strips whose key can
    still win, so neither the ids nor the previous row enter the lower bound."""
    bx = xadj_bits // 8
    fixed = steps * (8 + 2 * bx) + n * (8 + 2 * bx)
    if app != "node2vec" or as_built:
        return 4 * scanned + fixed
    return 8 * scanned + 4 * prev_scanned + fixed


def cpu_baseline(g, args, budget_s=12.0, full=False):
    """Times the CPU golden walker (OpenMP over queries) on a seeded sample of the workload.
    `g` needs V, xadj, adj, weight, label (numpy arrays)."""
    sys.path.insert(0, os.path.join(ROOT, "tests"))
    import oracle_lib as O
    V = g.V
    rng = np.random.default_rng(4)
    app = APPS[args.app]
    kw = dict(d=args.d, group_mode=args.group or 64)
    if args.app == "metapath":
        kw["schema"] = [0, 1, 2, 3, 4]
    cores = O.lib().fwo_max_threads()
    n = 20000
    best = None
    while True:
        starts = rng.integers(0, V, n).astype(np.int32)
        t0 = time.perf_counter()
        _, steps, scanned, _ = O.graph_walk(g, app, starts, **kw)
        dt = time.perf_counter() - t0
        best = (steps / dt, n, dt, steps, scanned)
        if dt >= budget_s / 3 or n >= 2000000 or not full and dt >= 3.0:
            break
        n = int(min(2000000, max(2 * n, n * (budget_s * 0.8) / max(dt, 1e-3))))
    return {"value": best[0], "unit": "walk steps/s", "cores": cores, "kind": "port",
            "sample": "%d seeded-uniform start vertices of the same graph, d=%d, %.1f s, %d steps, %d scanned"
                      % (best[1], args.d, best[2], best[3], best[4])}


def workload_name(args):
    starts = "--all" if not args.queries else "%d uniform starts" % args.queries
    return "%s %s d=%d on R-MAT scale-%d ef%d (a=%s,b=.19,c=.19), f32 weights in [%s), int%d CSR" % (
        args.app, starts, args.d, args.scale, args.edge_factor, ("%.2f" % args.rmat_a).lstrip("0"),
        args.weights, args.xadj_bits)


def make_config(args, V, E, n, steps_per_pass, scanned_per_pass, world, device):
    """The `config` object of the JSON line: the same keys in both arms."""
    return {"workload": workload_name(args), "queries_per_gpu_per_step": n, "vertices": V, "edges": E,
            "walk_steps_per_pass": steps_per_pass, "scanned_per_pass": scanned_per_pass,
            "group_mode": args.group or 64,
            "parallelism": "queries sharded, graph replicated x%d" % world,
            "l2": "inputs larger than L2 (weights %.0f MB, results %.0f MB per pass)" % (
                4 * E / 1e6, 4 * n * (args.d + 1) / 1e6),
            "device": device}


def make_graph(fw, args, device):
    lo, hi = (float(x) for x in args.weights.split(","))
    return fw.rmat(args.scale, args.edge_factor << args.scale, a=args.rmat_a, weight_range=(lo, hi),
                   n_labels=5 if args.app == "metapath" else 0, xadj_bits=args.xadj_bits, device=device)


def start_vertices(V, n):
    return np.arange(n, dtype=np.int32) if n == V else \
        np.random.default_rng(4).integers(0, V, n).astype(np.int32)


# Child process of the reference arm: generates the workload's graph with this repo's generator,
# writes it in the reference's on-disk format and the start vertices beside it.  The measuring
# process itself never loads this repo's library.
_GRAPH_CHILD = """
import json, sys
sys.path.insert(0, %(root)r)
import bench, flowwalker_artifact_b200 as fw
args = bench.parse()
g = bench.make_graph(fw, args, 0 if %(gpu)r else -1)
g.save(%(prefix)r)
n = args.queries or g.V
bench.start_vertices(g.V, n).tofile(%(starts)r)
print("GRAPHJSON " + json.dumps({"V": g.V, "E": g.E, "n": n}))
"""


class _HostGraph:
    """The saved graph read back with numpy (for the CPU baseline of the reference arm)."""

    def __init__(self, prefix, bits, want_label):
        raw = np.fromfile(prefix + "_xadj.bin", dtype=np.uint8)
        self.V = int(np.frombuffer(raw[:4].tobytes(), dtype=np.int32)[0])
        self.xadj = np.frombuffer(raw[8:].tobytes(), dtype=np.int64 if bits == 64 else np.uint32)
        self.adj = np.fromfile(prefix + "_edge.bin", dtype=np.int32)
        self.weight = np.fromfile(prefix + "_weight.bin", dtype=np.float32) if os.path.exists(prefix + "_weight.bin") else None
        self.label = np.fromfile(prefix + "_label.bin", dtype=np.int32) if want_label else None
        self.E = len(self.adj)


def run_reference(args):
    """Reference arm.  When the reference's own CUDA walker was rebuilt for sm_100
    (oracle/_ref/ref_walk: its unmodified walk.cu / util.cu / headers behind a harness) and a
    GPU is present, this times THAT on the same graph and start vertices: `value` from its
    walk_test path (kernel only, the time the reference itself measures), `e2e` from its
    walk_batch path (pinned host result, copies inside its timed region).  The reference has
    no CPU implementation of the walk; `cpu_baseline` is the OpenMP port of the same semantics
    (the golden walker).  Without the binary or a GPU the port is the value too.  With N > 1 the
    reference still runs on one GPU (it has no multi-GPU path)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import tempfile
    have_gpu = _has_cuda()
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_walk")
    line = {"impl": "reference", "metric": "walk steps/sec", "unit": "walk steps/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
    with tempfile.TemporaryDirectory() as tmp:
        prefix = os.path.join(tmp, "g")
        sp = os.path.join(tmp, "starts.bin")
        code = _GRAPH_CHILD % {"root": ROOT, "gpu": have_gpu, "prefix": prefix, "starts": sp}
        res = subprocess.run([sys.executable, "-c", code] + sys.argv[1:], capture_output=True, text=True, timeout=1800)
        info = [json.loads(ln[10:]) for ln in res.stdout.splitlines() if ln.startswith("GRAPHJSON ")]
        if res.returncode != 0 or not info:
            print(json.dumps({"impl": "reference", "unavailable": "graph generation failed: " + (res.stderr or res.stdout)[-200:].replace("\n", " ")}))
            return
        V, E, n = info[0]["V"], info[0]["E"], info[0]["n"]
        g = _HostGraph(prefix, args.xadj_bits, args.app == "metapath")
        cpu = cpu_baseline(g, args, budget_s=12.0, full=True)
        done = False
        if have_gpu and os.path.exists(ref_bin) and args.xadj_bits == 32:
            cmd = [ref_bin, prefix, args.app, str(args.d), sp, str(n), "-", "0.2", "2.0", "0.5"]
            if args.app == "metapath":
                cmd.append("0,1,2,3,4")
            out = {}
            for mode in ("0", "1"):
                env = dict(os.environ, FW_REF_REPEAT=str(args.warmup + args.steps), FW_REF_BATCH=mode)
                try:
                    res = subprocess.run(cmd, capture_output=True, text=True, timeout=1500, env=env)
                    recs = [json.loads(ln[8:]) for ln in res.stdout.splitlines() if ln.startswith("REFJSON ")]
                    if res.returncode == 0 and len(recs) == args.warmup + args.steps:
                        out[mode] = recs[args.warmup:]
                    else:
                        line.setdefault("errors", []).append((res.stdout + res.stderr)[-300:])
                except Exception as exc:  # noqa: BLE001
                    line.setdefault("errors", []).append(repr(exc)[:300])
            if "0" in out:
                ms = sum(r["ref_ms"] for r in out["0"])
                st = sum(r["steps"] for r in out["0"])
                sc = sum(r.get("scanned", 0) for r in out["0"])
                line.update({"value": st / (ms * 1e-3), "ms_per_step": ms / args.steps,
                             "config": make_config(args, V, E, n, st // args.steps, sc // args.steps, 1,
                                                   "one B200: the reference's CUDA walker rebuilt for sm_100, its own "
                                                   "timer around its kernel (walk_test)")})
                if "1" in out:
                    ms1 = sum(r["ref_ms"] for r in out["1"])
                    st1 = sum(r["steps"] for r in out["1"])
                    line["e2e"] = {"value": st1 / (ms1 * 1e-3), "unit": "walk steps/s", "h2d_bytes_per_step": 4 * n,
                                   "d2h_bytes_per_step": 4 * n * (args.d + 1), "ms_per_step": ms1 / args.steps,
                                   "timed": "the reference's walk_batch timer (copies included)"}
                else:
                    line["e2e"] = {"value": line["value"], "unit": "walk steps/s", "h2d_bytes_per_step": 0,
                                   "d2h_bytes_per_step": 0}
                done = True
        if not done:
            why = "64-bit row offsets do not fit the reference's edge_t" if args.xadj_bits == 64 else \
                "reference binary or GPU unavailable"
            line.update({"value": cpu["value"], "ms_per_step": None,
                         "config": make_config(args, V, E, n, None, None, 1, "host CPU (OpenMP port; %s)" % why),
                         "e2e": {"value": cpu["value"], "unit": "walk steps/s", "h2d_bytes_per_step": 0,
                                 "d2h_bytes_per_step": 0}})
        line["cpu_baseline"] = cpu
    print(json.dumps(line))


def _has_cuda():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def bind_near_gpu(torch, local):
    """Runs this rank on the CPUs next to its GPU (sysfs local_cpulist of the GPU's PCI function,
    within the CPUs the process may use), so that the page-locked buffers it allocates afterwards
    sit on that NUMA node and the copy threads do not cross the socket link.  Returns a short
    record for the JSON line; leaves everything alone when the topology is not visible."""
    try:
        p = torch.cuda.get_device_properties(local)
        bdf = "%04x:%02x:%02x.0" % (p.pci_domain_id, p.pci_bus_id, p.pci_device_id)
        base = "/sys/bus/pci/devices/" + bdf
        with open(base + "/local_cpulist") as f:
            text = f.read().strip()
        node = open(base + "/numa_node").read().strip() if os.path.exists(base + "/numa_node") else "?"
        cpus = set()
        for part in text.split(","):
            if "-" in part:
                a, b = part.split("-")
                cpus.update(range(int(a), int(b) + 1))
            elif part:
                cpus.add(int(part))
        allowed = os.sched_getaffinity(0)
        use = cpus & allowed
        if not use or use == allowed:
            return {"bound": False, "node": node, "why": "nothing to narrow (%d local of %d allowed CPUs)" % (len(use), len(allowed))}
        os.sched_setaffinity(0, use)
        return {"bound": True, "node": node, "cpus": len(use), "of": len(allowed)}
    except Exception as exc:  # noqa: BLE001
        return {"bound": False, "why": repr(exc)[:120]}


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    import flowwalker_artifact_b200 as fw
    from flowwalker_artifact_b200 import multi

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the walk engine has no CPU path")
    torch.cuda.set_device(local)
    numa = {"bound": False, "why": "--no-numa"} if args.no_numa else bind_near_gpu(torch, local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    g = make_graph(fw, args, local)
    eng = fw.Engine(g, local)
    eng.set_sharing(args.sharing)
    eng.set_hub_batching(args.hub_batching)
    eng.set_early_delivery(args.early_delivery)
    V = g.V
    n = args.queries or V
    D = args.d + 1
    kw = dict(d=args.d, group_mode=args.group)
    if args.app == "metapath":
        kw["schema"] = [0, 1, 2, 3, 4]
    starts_host = torch.from_numpy(start_vertices(V, n)).pin_memory()
    starts_dev = starts_host.cuda()
    result_dev = torch.empty((n, D), dtype=torch.int32, device="cuda")
    result_host = torch.empty((n, D), dtype=torch.int32).pin_memory()
    stream = torch.cuda.current_stream().cuda_stream

    def one(step_idx, host):
        prm = fw.make_params(APPS[args.app], seed=1337, query_id_base=(rank + world * step_idx) * n, **kw)
        if host:
            st = fw.WalkStats()
            # double-buffered batches: the result of one travels to the host while the next walks
            per_batch = (n + args.e2e_batches - 1) // args.e2e_batches
            rc = fw.lib().fw_walk_batch_into(eng._h, prm[0], starts_host.data_ptr(), n, per_batch, 512,
                                             result_host.data_ptr(), st, None)
            if rc:
                raise RuntimeError(fw.lib().fw_last_error())
            return st
        return eng.walk_device(prm, starts_dev.data_ptr(), n, result_dev.data_ptr(), stream=stream)

    def sync_all():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(host):
        for i in range(args.warmup):
            one(i, host)
        sync_all()
        sampler = ClockSampler(local)
        if rank == 0:
            sampler.start()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        steps = scanned = 0
        kernel_ms = 0.0
        status = 0
        launches = 0
        t0 = time.perf_counter()
        ev0.record()
        for i in range(args.steps):
            st = one(args.warmup + i, host)
            steps += st.steps
            scanned += st.scanned
            kernel_ms += st.device_ms
            status |= st.device_status
            launches += st.launches
        ev1.record()
        sync_all()
        wall_ms = (time.perf_counter() - t0) * 1e3
        ms = ev0.elapsed_time(ev1) if not host else wall_ms
        clocks = sampler.stop() if rank == 0 else None
        t = torch.tensor([ms, kernel_ms], dtype=torch.float64, device="cuda")
        c = torch.tensor([steps, scanned, launches, status], dtype=torch.int64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            status_t = c[3:].clone()
            dist.all_reduce(c, op=dist.ReduceOp.SUM)
            dist.all_reduce(status_t, op=dist.ReduceOp.MAX)
            c[3] = status_t[0]
        return dict(ms=float(t[0]), kernel_ms=float(t[1]), steps=int(c[0]), scanned=int(c[1]),
                    launches=int(c[2]), status=int(c[3]), clocks=clocks)

    def d2h_only():
        """Plain copy of the walk table to the page-locked host buffer, all ranks at once:
        what the host side of the end-to-end leg can take, in GB/s per rank (slowest rank)."""
        sync_all()
        ev0, ev1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        ev0.record()
        for _ in range(3):
            result_host.copy_(result_dev, non_blocking=True)
        ev1.record()
        torch.cuda.synchronize()
        t = torch.tensor([ev0.elapsed_time(ev1) / 3], dtype=torch.float64, device="cuda")
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return 4 * n * D / (float(t[0]) * 1e-3) / 1e9

    def strong_leg(n_job, interleaved, reps):
        """One job of n_job queries (query i starts at vertex i mod V) partitioned over the ranks;
        returns every rank's kernel time per pass, the job's walk steps, and this rank's rows."""
        if interleaved:
            ids = np.arange(rank, n_job, world, dtype=np.int64)
            base, stride = rank, world
        else:
            lo, hi = multi.shard_range(n_job, rank, world)
            ids = np.arange(lo, hi, dtype=np.int64)
            base, stride = lo, 1
        m = len(ids)
        st_dev = torch.from_numpy((ids % V).astype(np.int32)).cuda()
        out = result_dev[:m] if m <= n else torch.empty((m, D), dtype=torch.int32, device="cuda")
        ms = 0.0
        steps = 0
        for i in range(1 + reps):  # one untimed pass first
            sync_all()
            prm = fw.make_params(APPS[args.app], seed=4242, query_id_base=base, query_id_stride=stride, **kw)
            st = eng.walk_device(prm, st_dev.data_ptr(), m, out.data_ptr(), stream=stream)
            if i:
                ms += st.device_ms
                steps += st.steps
        mine = torch.tensor([ms / reps], dtype=torch.float64, device="cuda")
        every = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(every, mine)
        tot = torch.tensor([steps // reps], dtype=torch.int64, device="cuda")
        dist.all_reduce(tot, op=dist.ReduceOp.SUM)
        per_rank = [float(x[0]) for x in every]
        return per_rank, int(tot[0]), ids, out

    def parity_sample(ids, out, count=256):
        """Checker leg, outside every timed region: `count` of this rank's rows of the job just
        walked against the CPU golden walker (walks are keyed by query id, so any subset compares
        bit for bit)."""
        sys.path.insert(0, os.path.join(ROOT, "tests"))
        import oracle_lib as O
        pick = np.linspace(0, len(ids) - 1, num=min(count, len(ids)), dtype=np.int64)
        rows = out[torch.from_numpy(pick).cuda()].cpu().numpy()
        okw = {k: v for k, v in kw.items() if k != "group_mode"}
        ok = True
        for j, i in enumerate(pick.tolist()):
            qid = int(ids[i])
            ref = O.graph_walk(g, APPS[args.app], np.array([qid % V], dtype=np.int32), seed=4242,
                               query_id_base=qid, group_mode=args.group or 64, threads=1, **okw)[0]
            ok = ok and bool((ref[0] == rows[j]).all())
        flag = torch.tensor([1 if ok else 0], dtype=torch.int64, device="cuda")
        dist.all_reduce(flag, op=dist.ReduceOp.MIN)
        return "ok" if int(flag[0]) else "MISMATCH"

    dev = timed(host=False)
    e2e = None if args.no_e2e else timed(host=True)
    copy_gbs = None if args.no_e2e else d2h_only()
    if dev["status"]:
        raise SystemExit("device status %d reported by the walk kernel" % dev["status"])

    strong = None
    if world > 1 and not args.no_strong:
        strong = {"note": "one job partitioned over the ranks; per-rank CUDA-event kernel time per pass; "
                          "efficiency = one GPU's time for the whole job (this run's full pass of V queries, "
                          "times R for the R V job) / (R x slowest rank)"}
        one_gpu_ms_per_V = dev["kernel_ms"] / args.steps  # slowest rank's full pass, V queries on one GPU
        reps = max(3, args.steps)
        for name, n_job in (("job_V", V), ("job_RV", world * V)):
            leg = {"queries": n_job}
            for layout in ("contiguous", "interleaved"):
                per_rank, steps, ids, out = strong_leg(n_job, layout == "interleaved", reps)
                mx, mean = max(per_rank), sum(per_rank) / len(per_rank)
                leg[layout] = {"ms_per_rank": [round(x, 3) for x in per_rank], "ms_max": mx, "ms_mean": mean,
                               "imbalance": mx / mean, "steps_per_s": steps / (mx * 1e-3),
                               "efficiency_vs_n1": one_gpu_ms_per_V * (n_job / V) / (world * mx)}
                if name == "job_RV":
                    leg[layout]["parity_sample"] = parity_sample(ids, out)
            strong[name] = leg

    if rank == 0:
        peak, peak_kind = measured_peak()
        total_queries = n * world * args.steps
        launches = args.steps * world
        abytes = algorithmic_bytes(args.app, dev["scanned"], dev["steps"], total_queries, g.xadj_bits)
        per_launch_bytes = abytes / launches
        per_launch_ms = dev["kernel_ms"] / args.steps
        achieved = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9
        rev = fw.lib().fw_kernel_revision().decode()
        prof = PROFILED.get((args.app, args.scale, args.edge_factor, args.d, args.group or 64))
        per_pass_launches = dev["launches"] / launches
        roof = {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                "peak_source": peak_kind + " copy bandwidth",
                "kernel": "walk_kernel" if per_pass_launches == 1 else
                          "walk_kernel + hub_kernel: a hub-batched pass is a series of launches (%.0f per pass, plan and "
                          "scatter kernels included); bytes and time are those of the whole pass" % per_pass_launches,
                "kernel_revision": rev, "launches_per_pass": per_pass_launches,
                "algorithmic_bytes_per_launch": per_launch_bytes, "kernel_ms_per_launch": per_launch_ms,
                "algorithmic_bytes": "4 B per neighbour of every row stepped from, as if every walker swept its row itself "
                                     "(walkers that share a sweep read the row once, so the bytes moved are fewer)"}
        if args.app == "node2vec":
            built = algorithmic_bytes(args.app, dev["scanned"], dev["steps"], total_queries, g.xadj_bits,
                                      as_built=True) / launches
            roof["note"] = ("node2vec: achieved/frac count 8 B per candidate (weight + neighbour id) but leave out the "
                            "scope table's 4 B x sum deg(prev) term, which the engine does not count on the device; "
                            "as_built_* is the minimum of the engine as written: 4 B per candidate (its sweep reads "
                            "weights only)")
            roof["as_built_bytes_per_launch"] = built
            roof["as_built_achieved"] = built / (per_launch_ms * 1e-3) / 1e9
            roof["as_built_frac"] = roof["as_built_achieved"] / peak
        if prof and prof["kernel_revision"] == rev:
            traffic = prof["dram_per_algorithmic_byte"] * per_launch_bytes
            roof.update({"traffic": traffic, "traffic_source": "ncu dram bytes of a " + prof["captured_on"] +
                         ", scaled by algorithmic bytes",
                         "dram_frac": traffic / (per_launch_ms * 1e-3) / 1e9 / peak,
                         "issue_active": prof["issue_active"], "l2_hit_rate": prof["l2_hit_rate"],
                         "warp_instructions_per_step": prof["instructions_per_step"],
                         "limited_by": "instruction issue and latency, not HBM: shared sweeps and L2-resident hub rows keep "
                                       "DRAM traffic far below the algorithmic bytes, so frac exceeds 1"})
        else:
            roof.update({"traffic": None, "traffic_source": "no ncu capture of this workload on kernel revision " + rev
                         if not prof else "the ncu capture of this workload is of kernel revision %s, not %s"
                         % (prof["kernel_revision"], rev)})
        line = {
            "metric": "walk steps/sec", "value": dev["steps"] / (dev["ms"] * 1e-3), "unit": "walk steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev["ms"] / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": make_config(args, V, g.E, n, dev["steps"] // launches, dev["scanned"] // launches, world,
                                  "B200 x%d, this engine" % world),
            "gpu_launches": dev["launches"],
            "clocks": dev["clocks"],
            "roofline": roof,
        }
        if e2e:
            line["e2e"] = {"value": e2e["steps"] / (e2e["ms"] * 1e-3), "unit": "walk steps/s",
                           "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 4 * n * D,
                           "ms_per_step": e2e["ms"] / args.steps, "clocks": e2e["clocks"],
                           "d2h_only_gbs_per_rank": copy_gbs, "numa": numa,
                           "launches": e2e["launches"], "kernel_ms_per_step": e2e["kernel_ms"] / args.steps,
                           "early_delivery": "on: rows of ended walks are written to the page-locked host table by "
                                             "deliver_kernel during the series (its launches are counted in `launches`)"
                                             if args.early_delivery != 0 and e2e["launches"] > dev["launches"]
                                             else "off: one copy of the table after the last launch"}
        if strong:
            line["strong"] = strong
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(g, args, full=True)
        print(json.dumps(line))
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
