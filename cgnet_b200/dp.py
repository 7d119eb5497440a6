"""Data-parallel plumbing: the batch is sharded over one process per GPU and the only exchange is the gradient
all-reduce after the backward pass (the reference itself is single-GPU; its layer couples samples only through the
weight gradient and the fragment-norm statistics, and the statistics stay rank-local here).

The collective is torch.distributed's (NCCL over NVLink on GPUs, gloo on CPU for tests); this module only packs the
gradients into a few flat buckets so that small layers cost one launch instead of one per parameter, and
(``GradientAverager``) starts a bucket's collective from inside the backward pass as soon as its last gradient exists,
so that only the first layer's bucket is exposed after the backward pass.
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


class GradientAverager:
    """Averages (or sums) gradients over the process group, overlapped with the backward pass.

    The parameters are bucketed in reverse registration order, the order in which a backward pass produces their
    gradients.  A hook on every parameter counts the bucket down; the hook that completes a bucket packs it and
    starts its all-reduce asynchronously, on the stream the backward pass runs on, so later backward kernels
    overlap it.  ``finish()`` (call it after ``backward()``) starts what is still open, waits for every collective
    and scatters the results back into ``.grad`` with one multi-tensor copy per bucket.

    With ``overlap=False`` there are no hooks: ``finish()`` packs each bucket and runs its all-reduce on the
    current stream (no hop to the collective library's own stream), which is the cheaper choice when the gradients
    are small and the backward kernels fill every SM.

    Every rank must construct it over the same parameter list and produce gradients for the same parameters.
    With a single process (or no process group) the object does nothing.
    """

    def __init__(self, parameters, group=None, average=True, bucket_bytes=1 << 20, overlap=True):
        self.group = group
        self.average = average
        self.active = dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1
        self.world = dist.get_world_size(group) if self.active else 1
        self.collectives = 0
        self._buckets, self._handles, self._launched = [], [], []
        if not self.active:
            return
        params = [p for p in parameters if p.requires_grad]
        cur, size = [], 0
        for p in reversed(params):
            n = p.numel() * p.element_size()
            if cur and (size + n > bucket_bytes or p.dtype != cur[0].dtype or p.device != cur[0].device):
                self._buckets.append(cur)
                cur, size = [], 0
            cur.append(p)
            size += n
        if cur:
            self._buckets.append(cur)
        self._pending = [len(b) for b in self._buckets]
        self._started = [False] * len(self._buckets)
        self.overlap = overlap
        if overlap:
            for i, b in enumerate(self._buckets):
                for p in b:
                    self._handles.append(p.register_post_accumulate_grad_hook(self._make_hook(i)))
        backend = dist.get_backend(group)
        self._avg_op = average and backend == "nccl"      # gloo has no AVG: sum, then divide

    def _make_hook(self, i):
        def hook(_param):
            self._pending[i] -= 1
            if self._pending[i] == 0:
                self._start(i)
        return hook

    def _start(self, i):
        if self._started[i]:
            return
        self._started[i] = True
        bucket = [p for p in self._buckets[i] if p.grad is not None]
        if not bucket:
            return
        flat = torch.cat([p.grad.reshape(-1) for p in bucket])
        op = dist.ReduceOp.AVG if self._avg_op else dist.ReduceOp.SUM
        work = dist.all_reduce(flat, op=op, group=self.group, async_op=self.overlap)
        self._launched.append((bucket, flat, work))
        self.collectives += 1

    def finish(self):
        """Wait for the step's collectives, write the reduced gradients back; returns the number issued this step."""
        if not self.active:
            return 0
        for i in range(len(self._buckets)):
            self._start(i)
        for bucket, flat, work in self._launched:
            if work is not None:
                work.wait()
            if self.average and not self._avg_op:
                flat.div_(self.world)
            views, off = [], 0
            for p in bucket:
                n = p.grad.numel()
                views.append(flat[off:off + n].view_as(p.grad))
                off += n
            torch._foreach_copy_([p.grad for p in bucket], views)
        n = len(self._launched)
        self._launched = []
        self._pending = [len(b) for b in self._buckets]
        self._started = [False] * len(self._buckets)
        return n

    def remove(self):
        """Detach the hooks (the object is inert afterwards)."""
        for h in self._handles:
            h.remove()
        self._handles = []
        self.active = False


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
