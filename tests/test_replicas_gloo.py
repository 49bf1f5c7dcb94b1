"""The N > 1 host logic on CPU: two gloo ranks shard the synthetic work, run the
oracle on their shard, and reduce times (max) and counters (sum) as bench.py
does over NCCL."""
import os
import socket
import sys

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    p = s.getsockname()[1]
    s.close()
    return p


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      LOCAL_RANK=str(rank))
    from omoknuni_small_b200 import replicas, synth
    from oracle import capi as oracle
    dist.init_process_group("gloo", rank=rank, world_size=world)
    assert replicas.rank_info() == (rank, world, rank)
    # each rank selects on its own shard of trees (seeded by rank, not by world size)
    t = synth.make_selection_tree(256, 225, seed=replicas.shard_seed(7, rank))
    sel = oracle.puct_select(t, c_puct=1.5, vl_value=3, apply_vl=True)
    times = replicas.max_over_ranks(dist, [10.0 + rank, 5.0 - rank])
    counters = replicas.sum_counters(dist, {"selections": len(sel), "evals": 100 * (rank + 1)})
    lo, hi = replicas.shard_range(1001, rank, world)
    np.savez(os.path.join(out_dir, f"r{rank}.npz"), sel=sel, times=times, sels=counters["selections"],
             evals=counters["evals"], lo=lo, hi=hi)
    dist.barrier()
    dist.destroy_process_group()


def test_two_ranks_shard_and_reduce(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    r = [np.load(tmp_path / f"r{i}.npz") for i in range(world)]
    for x in r:
        assert list(x["times"]) == [11.0, 5.0]          # max over ranks
        assert int(x["sels"]) == 512 and int(x["evals"]) == 300
    assert not np.array_equal(r[0]["sel"], r[1]["sel"])  # different shards
    assert (int(r[0]["lo"]), int(r[0]["hi"]), int(r[1]["lo"]), int(r[1]["hi"])) == (0, 501, 501, 1001)
    # a shard's result does not depend on the world size: rank 1's shard recomputed alone
    sys.path.insert(0, ROOT)
    from omoknuni_small_b200 import replicas, synth
    from oracle import capi as oracle
    t = synth.make_selection_tree(256, 225, seed=replicas.shard_seed(7, 1))
    assert np.array_equal(oracle.puct_select(t, c_puct=1.5, vl_value=3, apply_vl=True), r[1]["sel"])
    assert replicas.aggregate_throughput(1024, 10, 8, 5.0) == 8 * 1024 * 10 / 5e-3
