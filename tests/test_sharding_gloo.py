"""world_size-2 gloo run of the multi-GPU host logic on CPU: shard ranges, id-keyed streams
(the union of the shards equals the single run) and the final counter reduction.  The walker
used inside the ranks is the CPU golden walker -- no GPU here."""
import os
import sys

import numpy as np
import torch.multiprocessing as mp

import graphs
import oracle_lib as O
from flowwalker_artifact_b200 import multi


def test_shard_range_partitions():
    for n in (0, 1, 7, 100, 4194304):
        for world in (1, 2, 3, 8):
            spans = [multi.shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == n
            assert all(spans[i][1] == spans[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in spans]
            assert max(sizes) - min(sizes) <= 1


def _worker(rank, world, port, tmpdir):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = graphs.config1()
    starts = graphs.config1_starts(301)
    lo, hi = multi.shard_range(len(starts), rank, world)
    res, steps, scanned, _ = O.graph_walk(g, 0, starts[lo:hi], d=20, query_id_base=lo)
    # the interleaved assignment (ids rank, rank + world, ...) gives the same rows
    inter = O.graph_walk(g, 0, starts[rank::world], d=20, query_id_base=rank, query_id_stride=world)[0]
    full_ids = np.arange(len(starts))
    mine = full_ids[rank::world]
    in_range = (mine >= lo) & (mine < hi)
    assert (inter[in_range] == res[mine[in_range] - lo]).all()
    (tot_steps, tot_scanned), (tmax,) = multi.reduce_counters(dist, [steps, scanned], [10.0 + rank])
    allrows = multi.gather_rows(dist, res, len(starts), rank, world)
    if rank == 0:
        np.savez(os.path.join(tmpdir, "out.npz"), rows=allrows, steps=tot_steps, scanned=tot_scanned, tmax=tmax)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_reproduce_the_single_run(tmp_path):
    world, port = 2, 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(world, port, str(tmp_path)), nprocs=world, join=True)
    out = np.load(os.path.join(str(tmp_path), "out.npz"))
    g = graphs.config1()
    starts = graphs.config1_starts(301)
    full, steps, scanned, _ = O.graph_walk(g, 0, starts, d=20)
    assert (out["rows"] == full).all()
    assert int(out["steps"]) == steps and int(out["scanned"]) == scanned
    assert float(out["tmax"]) == 11.0
