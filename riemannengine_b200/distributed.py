"""Sample sharding and weight-gradient all-reduce for data-parallel runs.

The hot path shards by sample: the batch index is column 0 of every coordinate and no kernel-map
pair crosses samples, so each rank hashes, maps and convolves its own samples with no forward
communication. The one collective of a training step is a sum of the weight gradients, done as a
single flat (bucketed) all-reduce per step: NCCL over NVLink on GPUs, gloo in the CPU tests of
this host logic. The reference has no distributed code at all (its ``RiemannSyncBatchNorm`` is an
alias of the plain layer, engine/nn/normalization.hpp:36-37).
"""
from __future__ import annotations

from typing import Iterable, List, Optional, Sequence

import numpy as np
import torch
import torch.distributed as dist


def assign_samples(voxels_per_sample: Sequence[int], world_size: int) -> List[List[int]]:
    """Greedy longest-processing-time assignment of whole samples to ranks, balanced by voxel
    count. Returns, per rank, the sorted list of sample (batch) indices it owns."""
    order = sorted(range(len(voxels_per_sample)), key=lambda i: (-int(voxels_per_sample[i]), i))
    loads = [0] * world_size
    owned: List[List[int]] = [[] for _ in range(world_size)]
    for i in order:
        r = min(range(world_size), key=lambda j: (loads[j], j))
        owned[r].append(i)
        loads[r] += int(voxels_per_sample[i])
    return [sorted(o) for o in owned]


def shard_rows(coords: np.ndarray, rank: int, world_size: int) -> np.ndarray:
    """Row indices of ``coords`` [N, 1 + D] (batch index in column 0) that belong to ``rank``."""
    batch = np.asarray(coords)[:, 0]
    n_samples = int(batch.max()) + 1 if len(batch) else 0
    counts = np.bincount(batch, minlength=n_samples)
    mine = assign_samples(counts.tolist(), world_size)[rank]
    return np.nonzero(np.isin(batch, mine))[0]


def allreduce_gradients(params: Iterable[torch.nn.Parameter], group: Optional[dist.ProcessGroup] = None,
                        average: bool = False, bucket_bytes: int = 64 << 20) -> int:
    """Sum (or average) the gradients of ``params`` over the ranks with as few collectives as
    possible: gradients are packed into flat fp32 buckets of at most ``bucket_bytes``.

    The bucket layout is a function of the parameter list alone, so every rank issues the same
    collectives with the same lengths whatever happened locally: a parameter whose gradient is
    ``None`` on this rank (a rank that was given no sample, a layer that a step did not use)
    contributes zeros and receives the reduced value as its gradient. Parameters that do not
    require a gradient are skipped on every rank alike.
    Returns the number of collectives issued. A no-op outside an initialised process group."""
    if not (dist.is_available() and dist.is_initialized()):
        return 0
    world = dist.get_world_size(group)
    plist = [p for p in params if p.requires_grad]
    if world == 1 or not plist:
        return 0
    calls = 0
    bucket: List[torch.nn.Parameter] = []
    size = 0

    def flush():
        nonlocal bucket, size, calls
        if not bucket:
            return
        flat = torch.cat([(p.grad.reshape(-1).float() if p.grad is not None
                           else torch.zeros(p.numel(), dtype=torch.float32, device=p.device)) for p in bucket])
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
        if average:
            flat /= world
        off = 0
        for p in bucket:
            n = p.numel()
            piece = flat[off:off + n].view(p.shape)
            if p.grad is None:
                p.grad = piece.to(p.dtype).clone()
            else:
                p.grad.copy_(piece)
            off += n
        calls += 1
        bucket, size = [], 0

    for p in plist:
        nbytes = p.numel() * 4
        if bucket and size + nbytes > bucket_bytes:
            flush()
        bucket.append(p)
        size += nbytes
    flush()
    return calls


def merge_batch_stats(stats: torch.Tensor, count: int, group: Optional[dist.ProcessGroup] = None):
    """Batch-normalisation moments over all ranks from each rank's per-channel sums.

    ``stats`` is float64 [2, C] (sum, sum of squares over this rank's ``count`` rows). One
    all-reduce of 2C + 1 numbers (no-op without an initialised process group) gives the
    whole-batch moments, which is what a single-process run over the full batch computes: returns
    (mean [C], biased variance [C], total row count)."""
    flat = torch.cat([stats.reshape(-1).to(torch.float64),
                      torch.tensor([float(count)], dtype=torch.float64, device=stats.device)])
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    total = float(flat[-1].item())
    c = stats.size(1)
    denom = max(total, 1.0)
    mean = flat[:c] / denom
    var = (flat[c:2 * c] / denom - mean * mean).clamp_min_(0.0)
    return mean, var, int(total)


def allreduce_sum_(tensors: Sequence[torch.Tensor], group: Optional[dist.ProcessGroup] = None) -> None:
    """In-place sum over ranks of a few small tensors as ONE flat all-reduce (no-op on one rank)."""
    if not (dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1):
        return
    flat = torch.cat([t.reshape(-1).to(torch.float64) for t in tensors])
    dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group)
    pos = 0
    for t in tensors:
        n = t.numel()
        t.copy_(flat[pos:pos + n].reshape(t.shape).to(t.dtype))
        pos += n
