"""Data-parallel plumbing: the batch is sharded over one process per GPU and the only exchange is the gradient
all-reduce after the backward pass (the reference itself is single-GPU; its layer couples samples only through the
weight gradient and the fragment-norm statistics, and the statistics stay rank-local here).

The collective is torch.distributed's (NCCL over NVLink on GPUs, gloo on CPU for tests); this module only packs the
gradients into a few flat buckets so that small layers cost one launch instead of one per parameter.
"""
import torch
import torch.distributed as dist


def _buckets(params, bucket_bytes):
    cur, size, out = [], 0, []
    for p in params:
        n = p.grad.numel() * p.grad.element_size()
        if cur and (size + n > bucket_bytes or p.grad.dtype != cur[0].grad.dtype or p.grad.device != cur[0].grad.device):
            out.append(cur)
            cur, size = [], 0
        cur.append(p)
        size += n
    if cur:
        out.append(cur)
    return out


def allreduce_gradients(parameters, group=None, average=True, bucket_bytes=64 << 20):
    """Sum (or average) ``.grad`` of every parameter over the process group, in place.

    All buckets are launched asynchronously, then waited for in order, so the copies of bucket i+1 overlap the
    collective of bucket i.  Parameters without a gradient are skipped (every rank must skip the same ones).
    Returns the number of collectives issued.
    """
    if not dist.is_available() or not dist.is_initialized():
        return 0
    world = dist.get_world_size(group)
    if world == 1:
        return 0
    params = [p for p in parameters if p.grad is not None]
    pending = []
    for bucket in _buckets(params, bucket_bytes):
        flat = torch.cat([p.grad.reshape(-1) for p in bucket])
        work = dist.all_reduce(flat, op=dist.ReduceOp.SUM, group=group, async_op=True)
        pending.append((bucket, flat, work))
    for bucket, flat, work in pending:
        work.wait()
        if average:
            flat.div_(world)
        off = 0
        for p in bucket:
            n = p.grad.numel()
            p.grad.copy_(flat[off:off + n].view_as(p.grad))
            off += n
    return len(pending)


def broadcast_parameters(module, src=0, group=None):
    """Make every rank start from rank ``src``'s parameters and buffers."""
    if not dist.is_available() or not dist.is_initialized() or dist.get_world_size(group) == 1:
        return
    for t in list(module.parameters()) + list(module.buffers()):
        dist.broadcast(t.data, src=src, group=group)


def shard_batch(n_samples, rank, world):
    """Contiguous slice of a global batch owned by ``rank`` (sizes differ by at most one)."""
    base, rem = divmod(n_samples, world)
    start = rank * base + min(rank, rem)
    return slice(start, start + base + (1 if rank < rem else 0))
