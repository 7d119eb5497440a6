"""The data-parallel plumbing at world size 2 on CPU (gloo): bucketed gradient all-reduce, parameter broadcast, batch
sharding.  The CG kernels themselves need a GPU; here the 'model' is a small torch module whose gradients have a
closed form, so the test checks the exchange, not the layer."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, bucket_bytes, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cgnet_b200.dp import allreduce_gradients, broadcast_parameters, shard_batch
        torch.manual_seed(100 + rank)                      # ranks start different on purpose
        net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 3))
        broadcast_parameters(net, src=0)
        ref = [p.detach().clone() for p in net.parameters()]
        gathered = [torch.zeros_like(ref[0]) for _ in range(world)]
        dist.all_gather(gathered, ref[0])
        same_start = all(torch.equal(gathered[0], g) for g in gathered)

        torch.manual_seed(7)
        X = torch.randn(10, 6)
        sl = shard_batch(10, rank, world)
        loss = net(X[sl]).pow(2).sum()                     # sum over the rank's samples
        loss.backward()
        n = allreduce_gradients(net.parameters(), average=False, bucket_bytes=bucket_bytes)
        grads = [p.grad.clone() for p in net.parameters()]

        net2 = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Linear(5, 3))
        with torch.no_grad():
            for p, r in zip(net2.parameters(), ref):
                p.copy_(r)
        net2(X).pow(2).sum().backward()                    # the whole batch on one process
        ok = all(torch.allclose(g, p.grad, rtol=1e-5, atol=1e-6) for g, p in zip(grads, net2.parameters()))
        results[rank] = (same_start, ok, n, (sl.start, sl.stop))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bucket_bytes", [64 << 20, 64])
def test_gradient_allreduce_world2_gloo(bucket_bytes):
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), bucket_bytes, results), nprocs=world, join=True)
        out = dict(results)
    assert set(out) == {0, 1}
    for rank in range(world):
        same_start, ok, n, _ = out[rank]
        assert same_start, "broadcast_parameters left the ranks with different weights"
        assert ok, "all-reduced gradients differ from the single-process gradients of the whole batch"
        assert n == (1 if bucket_bytes > 1024 else 4)
    assert out[0][3] == (0, 5) and out[1][3] == (5, 10)


def _averager_worker(rank, world, port, bucket_bytes, overlap, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from cgnet_b200.dp import GradientAverager, broadcast_parameters, shard_batch
        torch.manual_seed(5)
        net = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
        unused = torch.nn.Parameter(torch.ones(4))         # never receives a gradient: its bucket must still close
        broadcast_parameters(net, src=0)
        params = list(net.parameters()) + [unused]
        avg = GradientAverager(params, average=True, bucket_bytes=bucket_bytes, overlap=overlap)
        net2 = torch.nn.Sequential(torch.nn.Linear(6, 5), torch.nn.Tanh(), torch.nn.Linear(5, 3))
        net2.load_state_dict(net.state_dict())
        ok, counts = True, []
        for step in range(3):                              # several steps: the countdown state must reset
            torch.manual_seed(20 + step)
            X = torch.randn(10, 6)
            sl = shard_batch(10, rank, world)
            for p in params:
                p.grad = None
            net(X[sl]).pow(2).sum().backward()
            counts.append(avg.finish())
            for p in net2.parameters():
                p.grad = None
            (net2(X).pow(2).sum() / world).backward()      # mean over ranks of per-rank sums
            ok = ok and all(torch.allclose(p.grad, q.grad, rtol=1e-5, atol=1e-6)
                            for p, q in zip(net.parameters(), net2.parameters()))
            ok = ok and unused.grad is None
        avg.remove()
        for p in params:
            p.grad = None
        net(X[sl]).pow(2).sum().backward()
        results[rank] = (ok, counts, avg.finish())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("bucket_bytes,overlap", [(1 << 20, True), (64, True), (64, False)])
def test_gradient_averager_world2_gloo(bucket_bytes, overlap):
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_averager_worker, args=(world, _free_port(), bucket_bytes, overlap, results), nprocs=world, join=True)
        out = dict(results)
    assert set(out) == {0, 1}
    for rank in range(world):
        ok, counts, after_remove = out[rank]
        assert ok, "averaged gradients differ from the single-process gradients of the whole batch"
        assert counts == [1 if bucket_bytes > 1024 else 4] * 3
        assert after_remove == 0


def test_single_process_is_a_noop():
    from cgnet_b200.dp import allreduce_gradients, shard_batch
    p = torch.nn.Parameter(torch.ones(3))
    p.grad = torch.full((3,), 2.0)
    assert allreduce_gradients([p]) == 0 and torch.equal(p.grad, torch.full((3,), 2.0))
    assert [shard_batch(10, r, 3) for r in range(3)] == [slice(0, 4), slice(4, 7), slice(7, 10)]
    from cgnet_b200.dp import GradientAverager
    avg = GradientAverager([p])
    assert not avg.active and avg.finish() == 0
