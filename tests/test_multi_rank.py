"""Multi-rank path on CPU (gloo, world size 2): the batch partition that bench.py uses to shard a workload over
GPUs, checked end to end - every rank computes its own sequences (here with the CPU oracle standing in for the
kernel), rank 0 reassembles the jagged output and compares it with the unsharded result."""
import os

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import hstu_oracle as O
from ops_rec_b200 import workloads as W


def _small_workload():
    rng = np.random.default_rng(5)
    L = rng.integers(1, 90, 11).astype(np.int64)
    T = np.minimum(rng.integers(0, 6, 11), L - 1).astype(np.int64)
    return W.Workload("small", 11, 2, 16, 96, L, T, rab="shared", dtype="fp32", value_scale=1.0)


def _worker(rank, world, port, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = _small_workload()
        kw_full = W.materialize(full, "cpu", seed=3)
        parts = W.partition_lpt(full.lengths, world)
        mine = parts[rank]
        off = full.offsets()
        rows = np.concatenate([np.arange(off[i], off[i + 1]) for i in mine]) if len(mine) else np.zeros(0, np.int64)
        sub = full.subset(mine)
        kw = dict(kw_full, q=kw_full["q"][rows], k=kw_full["k"][rows], v=kw_full["v"][rows],
                  seq_offset=torch.from_numpy(sub.offsets()), num_target=torch.from_numpy(sub.targets))
        out = O.hstu_jagged_forward(**kw)
        gathered = [None] * world
        dist.all_gather_object(gathered, (rows, out))
        dist.barrier()
        if rank == 0:
            total = torch.zeros_like(kw_full["q"])
            seen = np.zeros(full.tokens, dtype=np.int64)
            for r, o in gathered:
                total[r] = o
                seen[r] += 1
            ref = O.hstu_jagged_forward(**kw_full)
            q.put((bool((seen == 1).all()), float((total - ref).abs().max())))
    finally:
        dist.destroy_process_group()


def test_sharded_forward_reassembles_to_the_unsharded_result():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    covered, err = q.get(timeout=10)
    assert covered and err == 0.0


@pytest.mark.parametrize("world", [1, 2, 4, 8])
def test_partition_covers_and_balances(world):
    w = W.make_workload("cfg4")
    parts = W.partition_lpt(w.lengths, world)
    allidx = np.sort(np.concatenate(parts))
    assert np.array_equal(allidx, np.arange(w.batch))
    flop_imb, tok_imb = W.imbalance(w.lengths, parts)
    assert flop_imb < 1.001 and tok_imb < 1.05
    assert abs(sum(w.subset(p).flops() for p in parts) - w.flops()) < 1e-6 * w.flops()


def test_workload_figures_match_the_baseline_table():
    want = {"cfg1": (292, 3.13e6), "cfg2": (21147, 16.07e9), "cfg3": (21147, 16.05e9), "cfg4": (623976, 4.279e12),
            "cfg5": (1111243, 0.280e12)}
    for name, (tokens, flops) in want.items():
        w = W.make_workload(name)
        assert w.tokens == tokens
        assert abs(w.flops() - flops) / flops < 2e-3
    assert abs(W.make_workload("cfg4").bytes() - 5.11e9) / 5.11e9 < 2e-3
    assert abs(W.make_workload("cfg3").bytes() - 149.3e6) / 149.3e6 < 2e-3
