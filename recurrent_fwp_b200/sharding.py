"""Partition of the fast-weight path over ranks (one process per GPU).

Every (batch, head) pair is an independent recurrence with its own state, so
the path shards over the batch axis with no collective on the data path: rank r
owns a contiguous slice of batch rows, runs the same kernels on it, and keeps
the matching slice of every carried state.  The reference does the same split
with ``nn.DataParallel`` along the batch dimension (language_modeling/src/train.py:525-533).

The only cross-rank reduction in the whole path is the sum over the batch of the
recurrent delta net's parameter gradients (dR_q, dR_k, dR_v, dr_b); those are
ordinary parameter gradients and join the trainer's data-parallel all-reduce.
``gather_outputs`` exists for end-to-end checks that want the full output on
every rank; it is not part of the hot path.
"""
import torch
import torch.distributed as dist


def batch_slice(n_batch, rank, world_size):
    """Contiguous, balanced slice of ``range(n_batch)`` owned by ``rank``."""
    if not 0 <= rank < world_size:
        raise ValueError('rank %d outside world of %d' % (rank, world_size))
    base, extra = divmod(n_batch, world_size)
    start = rank * base + min(rank, extra)
    return slice(start, start + base + (1 if rank < extra else 0))


def shard(tensors, rank, world_size):
    """Slice a list of (N, ...) tensors (streams or states) along the batch axis."""
    return [None if t is None else t[batch_slice(t.shape[0], rank, world_size)] for t in tensors]


def gather_outputs(local, n_batch, group=None):
    """All-gather per-rank output slices (batch-major) into the full (N, ...) tensor on every rank."""
    world = dist.get_world_size(group)
    sizes = [batch_slice(n_batch, r, world) for r in range(world)]
    longest = max(s.stop - s.start for s in sizes)
    pad = torch.zeros((longest,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    pad[:local.shape[0]] = local
    parts = [torch.empty_like(pad) for _ in range(world)]
    dist.all_gather(parts, pad, group=group)
    return torch.cat([p[:s.stop - s.start] for p, s in zip(parts, sizes)], dim=0)


def reduce_parameter_grads(grads, group=None):
    """Sum the recurrent delta net's parameter gradients over ranks (they are sums over the batch)."""
    for g in grads:
        dist.all_reduce(g, op=dist.ReduceOp.SUM, group=group)
    return grads
