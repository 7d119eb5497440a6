"""The CG layer under a two-rank NCCL process group, one rank per GPU (skipped on a machine with fewer than two GPUs).

The layer shards over samples; the batch couples the samples only through the weight gradient (a sum over the batch)
and the fragment-norm statistics (which stay rank-local by design).  So two things must hold exactly as on one GPU:

  (i)  inference: the outputs of the rank-sharded batch, put back together, equal the one-GPU outputs bit for bit
       (per-sample arithmetic does not depend on which other samples share the batch);
  (ii) training without the fragment norm: the weight gradients of the shards, summed by the all-reduce, equal the
       one-GPU gradient of the whole batch (up to the order of the fp32 sum over samples: 1e-5 relative).

The children are plain processes that join the group over 127.0.0.1; every rank leaves only after its last collective
has completed.  NVLink in-switch reduction is switched off: nothing here needs it.
"""
import os
import socket

import numpy as np
import pytest
import torch
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world),
                      NCCL_NVLS_ENABLE="0")
    import torch.distributed as dist
    dev = torch.device("cuda", rank)
    torch.cuda.set_device(dev)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from cgnet_b200 import CGBN_cuda
        from cgnet_b200.dp import GradientAverager, broadcast_parameters, shard_batch
        lmax, taus, tau_out, B = 5, [4] * 6, [8] * 6, 70
        rng = np.random.RandomState(5)
        X = torch.tensor(rng.randn(B, sum(t * (2 * l + 1) for l, t in enumerate(taus)), 2).astype(np.float32), device=dev)
        sl = shard_batch(B, rank, world)
        out = {}

        # (i) inference with stored statistics
        torch.manual_seed(100 + rank)                       # ranks start different on purpose
        layer = CGBN_cuda(lmax, taus, tau_out, batchnorm=True, device=dev)
        broadcast_parameters(layer, src=0)
        layer.eval()
        with torch.no_grad():
            full = layer(X, straight_output=True)
            mine = layer(X[sl].contiguous(), straight_output=True)
        parts = [torch.empty(shard_batch(B, r, world).stop - shard_batch(B, r, world).start, *mine.shape[1:], device=dev)
                 for r in range(world)]
        dist.all_gather(parts, mine)                        # shard sizes are equal here (70 / 2)
        out["eval_equal"] = bool(torch.equal(torch.cat(parts, 0), full))

        # (ii) training without the fragment norm: all-reduced (summed) gW of the shards = gW of the whole batch
        torch.manual_seed(200 + rank)
        lay2 = CGBN_cuda(lmax, taus, tau_out, batchnorm=False, device=dev)
        broadcast_parameters(lay2, src=0)
        lay2.train()
        G = torch.tensor(rng.randn(B, sum(t * (2 * l + 1) for l, t in enumerate(tau_out)), 2).astype(np.float32), device=dev)
        (lay2(X, straight_output=True) * G).sum().backward()
        gW_full = lay2.bnWMM.W.grad.clone()
        lay2.bnWMM.W.grad = None
        avg = GradientAverager([lay2.bnWMM.W], average=False, overlap=False)
        (lay2(X[sl].contiguous(), straight_output=True) * G[sl]).sum().backward()
        n = avg.finish()
        torch.cuda.synchronize()
        err = float((lay2.bnWMM.W.grad - gW_full).norm() / gW_full.norm())
        out["gw_rel_err"], out["collectives"] = err, n
        lay2.cg.plan.check_status()
        results[rank] = out
        dist.barrier()
        torch.cuda.synchronize()
    finally:
        dist.destroy_process_group()


def test_layer_under_two_rank_nccl_group():
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    world = 2
    with mp.Manager() as mgr:
        results = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), results), nprocs=world, join=True)
        out = dict(results)
    assert set(out) == {0, 1}
    for r in range(world):
        assert out[r]["eval_equal"], "sharded inference differs from the one-GPU outputs"
        assert out[r]["gw_rel_err"] < 1e-5, out[r]
        assert out[r]["collectives"] == 1
