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
(start vertices copied in, the whole walk table copied out, eight double-buffered batches:
measured 105.5 / 103.8 / 104.2 / 108.3 ms per pass with 4 / 8 / 16 / 32 batches).
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
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--e2e-batches", type=int, default=8, help="double-buffered batches of the end-to-end leg")
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


# DRAM bytes per algorithmic byte of the DeepWalk config-2 launch, from the ncu capture summarised
# in profiles/walk_kernel_deepwalk_scale22_tma_ring_strip64.md (dram__bytes_read.sum + write.sum = 53.07 GB
# for 249.08 GB algorithmic on a 1,000,000-query launch of the same graph; both grow in proportion
# with the number of queries).  Only valid for that workload: other runs report traffic = null.
DRAM_PER_ALGORITHMIC_BYTE = 0.2131


def algorithmic_bytes(app, scanned, steps, n, xadj_bits):
    """Weights (or labels) read once per scanned neighbour, plus per step the chosen
    neighbour id, the two row bounds of the new vertex and the result cell, plus per
    query the start vertex, its row bounds and the first result cell.  node2vec also
    reads every candidate's neighbour id (its previous-row term is not counted here)."""
    bx = xadj_bits // 8
    per_edge = 8 if app == "node2vec" else 4
    return per_edge * scanned + steps * (8 + 2 * bx) + n * (8 + 2 * bx)


def cpu_baseline(g, args, budget_s=12.0, full=False):
    """Times the CPU golden walker (OpenMP over queries) on a seeded sample of the workload."""
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


def make_graph(fw, args, device):
    lo, hi = (float(x) for x in args.weights.split(","))
    return fw.rmat(args.scale, args.edge_factor << args.scale, a=args.rmat_a, weight_range=(lo, hi),
                   n_labels=5 if args.app == "metapath" else 0, xadj_bits=args.xadj_bits, device=device)


def run_reference(args):
    """Reference arm.  When the reference's own CUDA walker was rebuilt for sm_100
    (oracle/_ref/ref_walk: its unmodified walk.cu / util.cu / headers behind a harness) and a
    GPU is present, this times THAT on the same graph and start vertices: `value` from its
    walk_test path (kernel only, the time the reference itself measures), `e2e` from its
    walk_batch path (pinned host result, copies inside its timed region).  The reference has
    no CPU implementation of the walk; `cpu_baseline` is the OpenMP port of the same semantics
    (the golden walker).  Without the binary or a GPU the port is the value too."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import tempfile
    import flowwalker_artifact_b200 as fw
    have_gpu = _has_cuda()
    g = make_graph(fw, args, 0 if have_gpu else -1)
    ref_bin = os.path.join(ROOT, "oracle", "_ref", "ref_walk")
    line = {"impl": "reference", "metric": "walk steps/sec", "unit": "walk steps/s", "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic"}
    cpu = cpu_baseline(g, args, budget_s=12.0, full=True)
    done = False
    if have_gpu and os.path.exists(ref_bin):
        n = args.queries or g.V
        with tempfile.TemporaryDirectory() as tmp:
            prefix = os.path.join(tmp, "g")
            g.save(prefix)
            starts = np.arange(n, dtype=np.int32) if n == g.V else \
                np.random.default_rng(4).integers(0, g.V, n).astype(np.int32)
            sp = os.path.join(tmp, "starts.bin")
            starts.tofile(sp)
            cmd = [ref_bin, prefix, args.app, str(args.d), sp, str(n), "-", "0.2", "2.0", "0.5"]
            if args.app == "metapath":
                cmd.append("0,1,2,3,4")
            out = {}
            for mode in ("0", "1"):
                env = dict(os.environ, FW_REF_REPEAT=str(args.warmup + args.steps), FW_REF_BATCH=mode)
                try:
                    res = subprocess.run(cmd, capture_output=True, text=True, timeout=900, env=env)
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
                line.update({"value": st / (ms * 1e-3), "ms_per_step": ms / args.steps,
                             "config": {"workload": workload_name(args), "device": "B200, reference CUDA walker rebuilt for sm_100",
                                        "queries_per_step": n, "timed": "the reference's own timer around its kernel (walk_test)"}})
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
        line.update({"value": cpu["value"], "ms_per_step": None,
                     "config": {"workload": workload_name(args), "device": "host CPU (OpenMP port; reference binary unavailable)"},
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


def main():
    args = parse()
    if args.impl == "reference":
        run_reference(args)
        return
    import torch
    import torch.distributed as dist
    import flowwalker_artifact_b200 as fw

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the walk engine has no CPU path")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    g = make_graph(fw, args, local)
    eng = fw.Engine(g, local)
    V = g.V
    n = args.queries or V
    D = args.d + 1
    kw = dict(d=args.d, group_mode=args.group)
    if args.app == "metapath":
        kw["schema"] = [0, 1, 2, 3, 4]
    starts_host = torch.arange(n, dtype=torch.int32).pin_memory() if n == V else \
        torch.from_numpy(np.random.default_rng(4).integers(0, V, n).astype(np.int32)).pin_memory()
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

    dev = timed(host=False)
    e2e = None if args.no_e2e else timed(host=True)
    if dev["status"]:
        raise SystemExit("device status %d reported by the walk kernel" % dev["status"])

    if rank == 0:
        peak, peak_kind = measured_peak()
        total_queries = n * world * args.steps
        abytes = algorithmic_bytes(args.app, dev["scanned"], dev["steps"], total_queries, g.xadj_bits)
        per_launch_bytes = abytes / (args.steps * world)
        per_launch_ms = dev["kernel_ms"] / args.steps
        achieved = per_launch_bytes / (per_launch_ms * 1e-3) / 1e9
        line = {
            "metric": "walk steps/sec", "value": dev["steps"] / (dev["ms"] * 1e-3), "unit": "walk steps/s",
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev["ms"] / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": {"workload": workload_name(args), "queries_per_gpu_per_step": n,
                       "vertices": V, "edges": g.E, "walk_steps_per_pass": dev["steps"] // (args.steps * world),
                       "scanned_per_pass": dev["scanned"] // (args.steps * world),
                       "group_mode": args.group or 64, "parallelism": "queries sharded, graph replicated x%d" % world,
                       "l2": "inputs larger than L2 (weights %.0f MB, results %.0f MB per pass)" % (
                           4 * g.E / 1e6, 4 * n * D / 1e6)},
            "gpu_launches": dev["launches"],
            "clocks": dev["clocks"],
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s",
                         "frac": achieved / peak,
                         "traffic": (DRAM_PER_ALGORITHMIC_BYTE * per_launch_bytes
                                     if (args.app, args.scale, args.edge_factor, args.d) == ("deepwalk", 22, 16, 80) else None),
                         "traffic_source": "ncu dram bytes of a 1,000,000-query launch scaled by algorithmic bytes",
                         "peak_source": peak_kind + " copy bandwidth",
                         "kernel": "walk_kernel", "algorithmic_bytes_per_launch": per_launch_bytes,
                         "kernel_ms_per_launch": per_launch_ms},
        }
        if e2e:
            line["e2e"] = {"value": e2e["steps"] / (e2e["ms"] * 1e-3), "unit": "walk steps/s",
                           "h2d_bytes_per_step": 4 * n, "d2h_bytes_per_step": 4 * n * D,
                           "ms_per_step": e2e["ms"] / args.steps}
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(g, args, full=True)
        print(json.dumps(line))
    eng.close()
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
