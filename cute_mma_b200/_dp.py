"""Token-sharded data parallelism for Prism layers: one process per GPU, every rank owns a
contiguous slice of the token rows (M) and a full copy of B, R and bias; the only exchange step is
the sum of the parameter gradients (dR, dB, dbias) over ranks, done with ``torch.distributed``
all-reduce (NCCL over NVLink on GPUs, gloo on CPU for the tests).

The reference has no collective of its own: its training script wraps the model in
``DistributedDataParallel`` (integration/train.py:130-145, 299-300), which performs exactly this
all-reduce in bucket hooks.  Here the gradients of one layer are packed into one flat bucket per
dtype so that a layer costs one collective launch.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(M: int, rank: int, world: int) -> tuple[int, int]:
    """Row range [lo, hi) of ``rank`` when M token rows are split as evenly as possible."""
    base, rem = divmod(M, world)
    lo = rank * base + min(rank, rem)
    return lo, lo + base + (1 if rank < rem else 0)


def allreduce_grads(grads, group=None, average: bool = False, async_op: bool = False):
    """Sum (or average) the given gradient tensors over the ranks of ``group``, in place.

    Tensors of the same dtype travel in one flat bucket.  With ``async_op=True`` returns a
    callable that waits for the collectives and scatters the buckets back.
    """
    grads = [g for g in grads if g is not None]
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return (lambda: None) if async_op else None
    world = dist.get_world_size(group)
    by_dtype = {}
    for g in grads:
        by_dtype.setdefault(g.dtype, []).append(g)
    pending = []
    for dtype, ts in by_dtype.items():
        flat = torch.cat([t.reshape(-1) for t in ts]) if len(ts) > 1 else ts[0].reshape(-1)
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((work, flat, ts))

    def finish():
        for work, flat, ts in pending:
            work.wait()
            if average:
                flat.div_(world)
            if len(ts) > 1 or flat.data_ptr() != ts[0].data_ptr():
                off = 0
                for t in ts:
                    n = t.numel()
                    t.copy_(flat[off:off + n].view_as(t))
                    off += n

    if async_op:
        return finish
    finish()
    return None


def sync_module_grads(module: torch.nn.Module, group=None, average: bool = True) -> None:
    """All-reduce the ``.grad`` of every trainable parameter of ``module`` (DDP semantics)."""
    allreduce_grads([p.grad for p in module.parameters() if p.requires_grad and p.grad is not None],
                    group=group, average=average)
