"""Token-sharded data parallelism for Prism layers: one process per GPU, every rank owns a
contiguous slice of the token rows (M) and a full copy of B, R and bias; the only exchange step is
the sum of the parameter gradients (dR, dB, dbias) over ranks, done with ``torch.distributed``
all-reduce (NCCL over NVLink on GPUs, gloo on CPU for the tests).

The reference has no collective of its own: its training script wraps the model in
``DistributedDataParallel`` (integration/train.py:130-145, 299-300), which performs exactly this
all-reduce in bucket hooks.  Here the gradients of one layer are packed into one flat bucket per
dtype so that a layer costs one collective launch.

``PeerGradReducer`` is the exchange without a library collective, for the GPUs of one box: the gradients
are written as fp32 into a buffer every rank can address (symmetric memory) and one kernel of this
library per rank adds its slice over the ranks in rank order with plain loads over NVLink and stores the
result to every rank (``prism_peer_reduce``): one pass, bit-identical on every rank and run.
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


def sync_module_grads(module: torch.nn.Module, group=None, average: bool = True, reducer=None) -> None:
    """Sum (``average``: mean) the ``.grad`` of every trainable parameter of ``module`` over the ranks (DDP
    semantics): an NCCL / gloo all-reduce, or with ``reducer`` (``PeerGradReducer.for_module(module)``) the
    library's rank-order fp32 sum over peer memory."""
    params = [p for p in module.parameters() if p.requires_grad and p.grad is not None]
    if reducer is None:
        allreduce_grads([p.grad for p in params], group=group, average=average)
        return
    if [tuple(p.shape) for p in params] != reducer.shapes:
        raise ValueError("the reducer was built for another set of parameters")
    torch._foreach_copy_(reducer.inputs(), [p.grad for p in params])
    outs = reducer.reduce()
    torch._foreach_copy_([p.grad for p in params], outs)


class PeerGradReducer:
    """Sum of a fixed set of gradient tensors over the GPUs of one box through peer memory.

    ``shapes``: the gradients' shapes, in the order they are passed to ``stage``/``reduce``.  One fp32
    staging buffer and one result buffer (``out_dtype``) are allocated as symmetric memory on every rank
    (``torch.distributed._symmetric_memory``) and exchanged once; afterwards a reduction is: every rank
    writes its gradients into ``inputs()`` (fp32 views of its staging buffer: the kernels' fp32 gradient
    outputs can be copied or written there), calls ``reduce()``, and reads ``outputs()``.
    ``reduce`` = barrier over the ranks, ``prism_peer_reduce`` on the current stream, barrier: rank r adds
    slice r of all ranks' buffers in rank order (the same bits on every rank, every run) and stores it to
    every rank.  ``ctas`` bounds the kernel's grid so that it can run beside a persistent kernel that
    leaves it a few SMs.
    """

    def __init__(self, shapes, out_dtype=torch.bfloat16, device=None, group=None, ctas: int = 16, average: bool = False):
        import ctypes

        import torch.distributed._symmetric_memory as symm_mem

        from . import _lib
        self._lib = _lib
        self.group = group if group is not None else dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self.shapes = [tuple(s) for s in shapes]
        self.offsets, n = [], 0
        for s in self.shapes:
            self.offsets.append(n)
            cnt = 1
            for d in s:
                cnt *= d
            n += (cnt + 3) // 4 * 4          # every tensor starts on a 16-byte boundary
        self.numel = (n + 4 * self.world - 1) // (4 * self.world) * (4 * self.world)
        self.out_dtype = out_dtype
        self.out_code = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}[out_dtype]
        self.scale = (1.0 / self.world) if average else 1.0
        self.ctas = ctas
        self._stage = symm_mem.empty(self.numel, dtype=torch.float32, device=self.device)
        self._result = symm_mem.empty(self.numel, dtype=out_dtype, device=self.device)
        self._stage.zero_()
        self._h_in = symm_mem.rendezvous(self._stage, self.group.group_name)
        self._h_out = symm_mem.rendezvous(self._result, self.group.group_name)
        vp = ctypes.c_void_p
        self._in_ptrs = (vp * self.world)(*[vp(int(p)) for p in self._h_in.buffer_ptrs])
        self._out_ptrs = (vp * self.world)(*[vp(int(p)) for p in self._h_out.buffer_ptrs])

    @classmethod
    def for_module(cls, module: torch.nn.Module, average: bool = True, **kw):
        """A reducer for the gradients of ``module``'s trainable parameters (``sync_module_grads(reducer=...)``);
        results in fp32, ``average`` as in DistributedDataParallel."""
        params = [p for p in module.parameters() if p.requires_grad]
        kw.setdefault("out_dtype", torch.float32)
        kw.setdefault("device", params[0].device)
        return cls([tuple(p.shape) for p in params], average=average, **kw)

    def _views(self, flat):
        out = []
        for s, off in zip(self.shapes, self.offsets):
            cnt = 1
            for d in s:
                cnt *= d
            out.append(flat[off:off + cnt].view(s))
        return out

    def inputs(self):
        """fp32 views of this rank's staging buffer, one per gradient."""
        return self._views(self._stage)

    def outputs(self):
        """views of this rank's result buffer (the sums over all ranks), one per gradient."""
        return self._views(self._result)

    def stage(self, grads):
        """Copy (and widen to fp32) this rank's gradients into the staging buffer."""
        for dst, g in zip(self.inputs(), grads):
            dst.copy_(g)

    def reduce(self):
        """The exchange, on the current stream; returns ``outputs()``."""
        import ctypes
        stream = torch.cuda.current_stream(self.device)
        self._h_in.barrier(channel=0)      # every rank's gradients are in its staging buffer
        with torch.cuda.device(self.device):
            self._lib.check(self._lib.lib().prism_peer_reduce(
                self._in_ptrs, self._out_ptrs, self.world, self.rank, self.numel, self.out_code,
                ctypes.c_float(self.scale), self.ctas, ctypes.c_void_p(stream.cuda_stream)))
        self._h_out.barrier(channel=1)     # every slice has reached every rank; the staging buffers may be rewritten
        return self.outputs()
