"""world_size-2 gloo tests (CPU) of the multi-rank host logic: sample sharding and the bucketed
weight-gradient all-reduce."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from riemannengine_b200 import distributed as D


def test_assign_samples_is_a_balanced_partition():
    counts = [150, 90, 120, 30, 150, 60, 100, 100]
    for world in (1, 2, 4, 8):
        owned = D.assign_samples(counts, world)
        flat = sorted(i for o in owned for i in o)
        assert flat == list(range(len(counts)))
        loads = [sum(counts[i] for i in o) for o in owned]
        assert max(loads) - min(loads) <= max(counts)


def test_shard_rows_keeps_samples_whole():
    rng = np.random.default_rng(0)
    coords = np.concatenate([rng.integers(0, 5, (1000, 1)), rng.integers(0, 9, (1000, 3))], 1).astype(np.int32)
    rows = [D.shard_rows(coords, r, 2) for r in range(2)]
    assert sorted(np.concatenate(rows).tolist()) == list(range(1000))
    b0, b1 = set(coords[rows[0], 0].tolist()), set(coords[rows[1], 0].tolist())
    assert not (b0 & b1)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    params = [torch.nn.Parameter(torch.zeros(27, 8, 8)), torch.nn.Parameter(torch.zeros(8, 4, 16)),
              torch.nn.Parameter(torch.zeros(1, 16)), torch.nn.Parameter(torch.zeros(3))]
    for i, p in enumerate(params[:3]):
        p.grad = torch.full_like(p, float(rank + 1) * (i + 1))
    calls_one = D.allreduce_gradients(params)  # the parameter without a gradient anywhere reduces to zeros
    ok = all(torch.equal(p.grad, torch.full_like(p, 3.0 * (i + 1))) for i, p in enumerate(params[:3]))
    ok = ok and params[3].grad is not None and torch.equal(params[3].grad, torch.zeros(3))
    for i, p in enumerate(params[:3]):
        p.grad = torch.full_like(p, float(rank + 1))
    calls_many = D.allreduce_gradients(params, average=True, bucket_bytes=4096)
    ok = ok and all(torch.allclose(p.grad, torch.full_like(p, 1.5)) for p in params[:3])
    out[rank] = (ok, calls_one, calls_many)
    dist.barrier()
    dist.destroy_process_group()


def test_bucketed_allreduce_two_ranks_gloo():
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        for r in range(world):
            ok, calls_one, calls_many = out[r]
            assert ok
            assert calls_one == 1          # everything fits one bucket
            assert calls_many >= 2         # small buckets -> several collectives, same result


def _uneven_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    # rank 1 was given no sample: every gradient is None there; rank 0 left one layer unused
    params = [torch.nn.Parameter(torch.zeros(27, 4, 4)), torch.nn.Parameter(torch.zeros(5)),
              torch.nn.Parameter(torch.zeros(2, 2), requires_grad=False)]
    if rank == 0:
        params[0].grad = torch.full_like(params[0], 2.0)
    calls = D.allreduce_gradients(params, average=True)
    ok = calls == 1 and torch.equal(params[0].grad, torch.full_like(params[0], 1.0))
    ok = ok and torch.equal(params[1].grad, torch.zeros(5)) and params[2].grad is None
    out[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_allreduce_with_missing_gradients_on_one_rank_gloo():
    """Ranks whose gradients are None for some (or all) parameters still issue the same collective."""
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_uneven_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert all(out[r] for r in range(world))


def test_allreduce_is_noop_without_process_group():
    p = torch.nn.Parameter(torch.ones(3))
    p.grad = torch.ones(3)
    assert D.allreduce_gradients([p]) == 0
    assert torch.equal(p.grad, torch.ones(3))


def _stats_worker(rank, world, port, out):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(7)
    x = torch.randn(1000, 6, generator=g, dtype=torch.float64) * 2 + 1   # same full batch on every rank
    mine = x[:300] if rank == 0 else x[300:]                             # uneven shards
    stats = torch.stack([mine.sum(0), (mine * mine).sum(0)])
    mean, var, total = D.merge_batch_stats(stats, mine.size(0))
    ok = total == 1000 and torch.allclose(mean, x.mean(0)) and torch.allclose(var, x.var(0, unbiased=False))
    a, b = torch.full((6,), float(rank + 1)), torch.full((2, 3), 10.0 * (rank + 1))
    D.allreduce_sum_([a, b])
    ok = ok and torch.equal(a, torch.full((6,), 3.0)) and torch.equal(b, torch.full((2, 3), 30.0))
    out[rank] = bool(ok)
    dist.barrier()
    dist.destroy_process_group()


def test_batch_stats_merge_two_ranks_gloo():
    """Whole-batch moments from per-rank sums (the sync batch-norm exchange) equal the single-process moments."""
    world = 2
    with mp.Manager() as m:
        out = m.dict()
        mp.spawn(_stats_worker, args=(world, _free_port(), out), nprocs=world, join=True)
        assert all(out[r] for r in range(world))
    # one rank, no process group: plain moments
    x = torch.arange(12, dtype=torch.float64).reshape(4, 3)
    mean, var, total = D.merge_batch_stats(torch.stack([x.sum(0), (x * x).sum(0)]), 4)
    assert total == 4 and torch.allclose(mean, x.mean(0)) and torch.allclose(var, x.var(0, unbiased=False))
