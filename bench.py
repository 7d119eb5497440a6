#!/usr/bin/env python
"""Benchmark of the CG-layer hot path: samples/s of a CG network step.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--global-batch G]

Workloads (synthetic, seeded; `python bench.py --list` prints them):
  cgnet5_lmax10              5 CG layers, lmax 10, tau 1 -> 5, full pair list, fragment norm in training mode,
                             skip-concatenated l=0 invariants -> BatchNorm1d -> Linear(52,256) -> ReLU -> Linear(256,10)
                             -> log-softmax -> NLL; batch 100 per GPU; input coefficient (l, m) ~ complex N(0, 1/(2l+1)).
                             Forward + backward.  The default.
  cgnet6_lmax14_tau16        SphericalCNN_fast training step: 6 input channels, 6 CG layers of 16 channels, lmax 14, batch
                             64, head -> 55 classes, forward + backward + SGD update, gradients all-reduced over the ranks.
  mst_lmax20_tau32           4 CG layers, lmax 20, 32 channels, MST pair lists with the reference's full channel product,
                             batch 128, inference.   mst_lmax20_tau32_depthwise: the channel-wise product on the same pairs.
  fused_layer_lmax{10,20,30}_tau{16,32,64}   one fused layer, inference (batch per GPU stated in `config`).
  layer_lmax5                one CG layer, lmax 5, tau 8, batch 32 (the reference's CPU-runnable case), forward + backward.

One JSON line is printed by rank 0.  `value` is timed with CUDA events around each step with the inputs already in
HBM, the L2 flushed (a 256 MB write) between steps and outside the timed intervals; `e2e` repeats the measurement through
the public module call with the step's input copied from pinned host memory and the step's result read back to the
host inside the timed interval.  With N > 1 every rank processes its own batch (weak scaling; `--global-batch G` splits
a fixed batch instead: strong scaling) and a training step ends with the NCCL all-reduce of all gradients; times are
the maximum over ranks.  Beside the numbers of this library the line carries `reference_cuda` (the same step through
the reference project's own CUDA kernels on the same GPU, when its extension was built into oracle/_ref), `cpu_baseline`
(the CPU restatement of the reference's Python layer on a bounded sample) and, for the default workload, `lmax20` (a
short run of the lmax-20 workloads, so that one record holds both degrees the headline metric names).

`--impl reference` times the CPU restatement of the reference's own Python layer (oracle/cg_oracle.py, torch CPU ops
with all host threads) on the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import numpy as np  # noqa: E402
import torch  # noqa: E402

METRIC_TRAIN = "CG-net samples/sec (training step, forward+backward)"
METRIC_INFER = "CG-net samples/sec (inference forward)"
METRIC_LAYER = "fused CG layer samples/sec (inference forward)"


def _wl(kind, lmax, tau_in, tau, layers, batch, describe, classes=10, hidden=256, pairs="default", depthwise=False,
        front="flat", optimizer=None):
    return dict(kind=kind, lmax=lmax, tau_in=tau_in, tau=tau, layers=layers, batch=batch, classes=classes, hidden=hidden,
                pairs=pairs, depthwise=depthwise, front=front, optimizer=optimizer, describe=describe)


WORKLOADS = {
    "cgnet5_lmax10": _wl("train", 10, 1, 5, 5, 100, "5-layer CGNet classifier, lmax 10, 5 channels, batch 100, forward+backward"),
    "layer_lmax5": _wl("train", 5, 8, 8, 1, 32, "single CG layer, lmax 5, 8 channels, batch 32, forward+backward"),
    "cgnet2_lmax14_tau16": _wl("train", 14, 16, 16, 2, 64, "2 CG layers, lmax 14, 16 channels, batch 64, forward+backward"),
    "cgnet6_lmax14_tau16": _wl("train", 14, 6, 16, 6, 64,
                               "SphericalCNN_fast training step: 6 input channels, 6 CG layers of 16 channels, lmax 14, batch 64, "
                               "55 classes, forward+backward+SGD update", classes=55, front="fast", optimizer="sgd"),
    "mst_lmax20_tau32": _wl("infer_net", 20, 32, 32, 4, 128,
                            "4 CG layers, lmax 20, 32 channels, MST pair lists with the full channel product (the reference's "
                            "'mst' mode), batch 128, inference", pairs="mst"),
    "mst_lmax20_tau32_depthwise": _wl("infer_net", 20, 32, 32, 4, 128,
                                      "4 CG layers, lmax 20, 32 channels, MST pair lists with the channel-wise (depthwise) "
                                      "product, batch 128, inference", pairs="mst", depthwise=True),
}
# The single-layer throughput sweep: batch 1024 split over the GPUs in the configuration it comes from; here a batch per
# GPU that keeps one step between a millisecond and a second (the number is stated in `config`).
for _L, _t, _b in ((10, 16, 256), (10, 32, 128), (10, 64, 64), (20, 16, 64), (20, 32, 32), (20, 64, 16), (30, 16, 32), (30, 32, 16),
                   (30, 64, 8)):
    WORKLOADS[f"fused_layer_lmax{_L}_tau{_t}"] = _wl(
        "layer_infer", _L, _t, _t, 1, _b, f"one fused CG layer, lmax {_L}, {_t} channels, batch {_b} per GPU, inference forward", hidden=0)


def synth_batch(wl, seed, batch=None):
    """Seeded stand-in for spherical-harmonic coefficients of a band-limited function: variance 1/(2l+1) per degree.
    Flat layout (B, sum_l tau_in (2l+1), 2); the `fast` front end gets the same numbers as (B, C, (lmax+1)^2, 2)."""
    B = batch or wl["batch"]
    rng = np.random.RandomState(seed)
    if wl["front"] == "fast":
        scale = np.concatenate([np.full(2 * l + 1, 1.0 / np.sqrt(2.0 * (2 * l + 1))) for l in range(wl["lmax"] + 1)])
        x = (rng.randn(B, wl["tau_in"], (wl["lmax"] + 1) ** 2, 2) * scale[None, None, :, None]).astype(np.float32)
    else:
        parts = [rng.randn(B, wl["tau_in"] * (2 * l + 1), 2) / np.sqrt(2.0 * (2 * l + 1)) for l in range(wl["lmax"] + 1)]
        x = np.concatenate(parts, axis=1).astype(np.float32)
    y = rng.randint(0, wl["classes"], size=B).astype(np.int64)
    return x, y


def layer_taus(wl):
    L1 = wl["lmax"] + 1
    return [[wl["tau_in"]] * L1] + [[wl["tau"]] * L1 for _ in range(wl["layers"])]


def pair_list(wl):
    from cgnet_b200 import CGutils
    S = CGutils.SparseLtuples
    lt = S.compute_mst_ltuples(wl["lmax"]) if wl["pairs"] == "mst" else S.compute_default_ltuples(wl["lmax"])
    return S.sparse_rep_ltuples_sorted(lt)[0]


# ---------------------------------------------------------------------------------------------------------------
# algorithmic work per sample (forward), from the shapes alone
# ---------------------------------------------------------------------------------------------------------------
def layer_work(lmax, taus, tau_out, llls=None, depthwise=False):
    """CG-product flops 8 * sum over triples of tau_l1 tau_l2 nnz, mixing flops 8 * sum_l t_FF[l] tau_out[l] (2l+1), and
    the sizes the fused kernels' algorithmic bytes follow from (depthwise: tau_l1 channels per triple)."""
    from cgnet_b200 import CGutils
    if llls is None:
        llls = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(CGutils.SparseLtuples.compute_default_ltuples(lmax))[0]
    cg_flops = 0
    t_ff = np.zeros(lmax + 1, dtype=np.int64)
    cg_len = 0
    for l, l1, l2 in CGutils.SparseLtuples.get_iter(lmax, llls):
        # number of (m, m2) with |m| <= l, |m2| <= l2, |m - m2| <= l1
        nnz = sum(min(l2, m + l1) - max(-l2, m - l1) + 1 for m in range(-l, l + 1))
        ch = taus[l1] if depthwise else taus[l1] * taus[l2]
        cg_flops += 8 * ch * nnz
        t_ff[l] += ch
        cg_len += (2 * l + 1) * (2 * l2 + 1)
    n = 2 * np.arange(lmax + 1) + 1
    mix_flops = int(8 * (t_ff * np.asarray(tau_out) * n).sum())
    return dict(cg_flops=int(cg_flops), mix_flops=mix_flops, n_F=int((np.asarray(taus) * n).sum()),
                n_O=int((np.asarray(tau_out) * n).sum()), n_FF=int((t_ff * n).sum()), w_len=int((t_ff * np.asarray(tau_out)).sum()),
                sum_tff=int(t_ff.sum()), cg_len=int(cg_len))


# ---------------------------------------------------------------------------------------------------------------
# networks
# ---------------------------------------------------------------------------------------------------------------
class Net(torch.nn.Module):
    """The reference's classifier shape (MNIST/model.py:28-67, Shrec17/Shrec17_main_fast.py:64-124) on top of a CG
    network `cnn` with an `output_length`, dropout left out."""

    def __init__(self, cnn, wl, device):
        super().__init__()
        self.cnn = cnn
        n = cnn.output_length
        self.bm1 = torch.nn.BatchNorm1d(n)
        self.fc = torch.nn.Linear(n, wl["hidden"])
        self.final = torch.nn.Linear(wl["hidden"], wl["classes"])
        self.to(device)

    def forward(self, x):
        x = self.bm1(self.cnn(x))
        x = torch.relu(self.fc(x))
        return torch.log_softmax(self.final(x), dim=1)


def build_ours(wl, dev):
    """The workload's network on this library, and the parameters a training step updates."""
    from cgnet_b200 import CGBN_cuda, SphericalCNN, SphericalCNN_fast
    L1 = wl["lmax"] + 1
    sparse = wl["pairs"] == "mst"
    if wl["kind"] == "layer_infer":
        net = CGBN_cuda(wl["lmax"], [wl["tau_in"]] * L1, [wl["tau"]] * L1, batchnorm=True, sparse_flag=sparse, device=dev,
                        depthwise=wl["depthwise"])
        return net.eval()
    if wl["front"] == "fast":
        cnn = SphericalCNN_fast(wl["lmax"], [wl["tau"]] * L1, wl["layers"], skip_type=1, num_channels_input=wl["tau_in"],
                                sparse_flag=sparse, device=dev, depthwise=wl["depthwise"])
    else:
        cnn = SphericalCNN(wl["lmax"], layer_taus(wl), norm=True, skipconn=True, sparse_flag=sparse, device=dev,
                           depthwise=wl["depthwise"])
    if wl["kind"] == "infer_net":
        return cnn.eval()
    return Net(cnn, wl, dev).train()


class ClockSampler:
    """nvidia-smi clock / throttle-reason samples taken while the timed region runs."""

    def __init__(self, index):
        self.rows = []          # (host time when the line arrived, fields)
        self.proc = None
        self.index = index
        self.window = None      # (t0, t1) of the timed region on the host clock

    def start(self):
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits",
                                          "-lms", "50"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.12)
        self.proc.terminate()
        rows = [r for t, r in self.rows if self.window is None or self.window[0] <= t <= self.window[1] + 0.06]
        scope = "timed region"
        if not rows:   # the timed region was shorter than the sampling period: use the samples of the whole loaded run
            rows, scope = [r for _, r in self.rows], "warm-up + timed region"
        sm = [float(r[0]) for r in rows if r and r[0].replace(".", "").isdigit()]
        mx = [float(r[1]) for r in rows if len(r) > 1 and r[1].replace(".", "").isdigit()]
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        reasons = [n for i, n in enumerate(names) if any(len(r) > 4 + i and r[4 + i].lower().startswith("active") for r in rows)]
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None, "reasons": reasons,
                "samples": len(sm), "scope": scope}


# DRAM bytes of one launch (read + write) from the ncu captures summarised under profiles/, per (workload, kernel).
# They are measurements of a fixed build on a fixed shape, not computed here; a pair without a capture reports null.
NCU_TRAFFIC = {
    ("cgnet5_lmax10", "fused_grad_f"): 1.93e6,
    ("cgnet5_lmax10", "fused_grad_w"): 1.58e6,
    ("cgnet5_lmax10", "fused_stats"): 0.93e6,
    ("cgnet5_lmax10", "fused_fwd"): 1.27e6,
    ("fused_layer_lmax10_tau16", "fused_fwd_tensor"): 56.1e6,
}


class Runner:
    """One workload on this rank's GPU: network, batches, the step, and device-timed loops over it."""

    def __init__(self, wl_name, wl, dev, rank, world, batch, net=None):
        import torch.distributed as dist
        from cgnet_b200.dp import GradientAverager, broadcast_parameters
        self.wl_name, self.wl, self.dev, self.rank, self.world, self.B = wl_name, wl, dev, rank, world, batch
        self.dist = dist
        self.train = wl["kind"] == "train"
        torch.manual_seed(1234)
        np.random.seed(1234)
        self.net = build_ours(wl, dev) if net is None else net
        if world > 1 and self.train:
            broadcast_parameters(self.net)
        self.params = [p for p in self.net.parameters() if p.requires_grad]
        # gradients of the 5-layer network are 1.5 MB, of the 6-layer lmax-14 network 157 MB: one bucket either way, one
        # all-reduce on the compute stream after the backward pass (per-layer buckets started inside the backward pass
        # were measured slower at the small size: each collective takes SMs from the persistent backward kernels)
        self.averager = (GradientAverager(self.params, average=True, bucket_bytes=256 << 20, overlap=False)
                         if world > 1 and self.train else None)
        self.opt = torch.optim.SGD(self.params, lr=1e-3) if wl["optimizer"] == "sgd" else None
        self.n_batches = 4 if batch * self._sample_bytes() < (256 << 20) else 2
        host = [synth_batch(wl, 100 + rank * self.n_batches + i, batch) for i in range(self.n_batches)]
        self.dev_batches = [(torch.tensor(x, device=dev), torch.tensor(y, device=dev)) for x, y in host]
        self.pinned = [(torch.tensor(x).pin_memory(), torch.tensor(y).pin_memory()) for x, y in host]
        self.flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        self.loss_fn = torch.nn.NLLLoss()

    def _sample_bytes(self):
        wl = self.wl
        return 8 * wl["tau_in"] * (wl["lmax"] + 1) ** 2

    def step(self, x, y):
        if not self.train:
            with torch.no_grad():
                out = self.net(x, straight_output=True) if self.wl["kind"] == "layer_infer" else self.net(x)
                return out.reshape(out.shape[0], -1)[:, :8].sum()   # a small read-back value for the end-to-end pass
        for p in self.params:
            p.grad = None
        loss = self.loss_fn(self.net(x), y)
        loss.backward()
        if self.averager is not None:
            self.averager.finish()
        if self.opt is not None:
            self.opt.step()
        return loss

    def barrier(self):
        if self.world > 1:
            self.dist.barrier()
        torch.cuda.synchronize()

    def warm(self, n):
        for i in range(n):
            self.step(*self.dev_batches[i % self.n_batches])
        self.barrier()

    def timed(self, n_steps, e2e):
        """Sum of per-step device times (ms), maximum over ranks; L2 flush between steps, outside the timed intervals."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_steps)]
        self.barrier()
        for i in range(n_steps):
            self.flush.fill_(i & 0xFF)
            ev[i][0].record()
            if e2e:
                xh, yh = self.pinned[i % self.n_batches]
                x = xh.to(self.dev, non_blocking=True)
                y = yh.to(self.dev, non_blocking=True)
                self.step(x, y).item()    # device -> host read of the step's result, inside the timed interval
            else:
                self.step(*self.dev_batches[i % self.n_batches])
            ev[i][1].record()
        self.barrier()
        total = sum(a.elapsed_time(b) for a, b in ev)
        t = torch.tensor([total], dtype=torch.float64, device=self.dev)
        if self.world > 1:
            self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def check_plans(self):
        """Raise if any tensor-core kernel of the network gave up on a bounded wait during the run."""
        for m in self.net.modules():
            plan = getattr(getattr(m, "cg", None), "plan", None)
            if plan is not None:
                plan.check_status()

    def h2d_bytes(self):
        return int(self.pinned[0][0].numel() * 4 + self.pinned[0][1].numel() * 8)


def time_reference_cuda(wl, dev, batch, steps):
    """The same step through the reference project's own CUDA kernels (its extension compiled unmodified for sm_100a
    into oracle/_ref), CUDA events, same GPU, same process.  Returns a dict, or {"unavailable": why}."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    try:
        import ref_cuda_driver as refdrv
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"driver import failed: {e}"}
    if not refdrv.available():
        return {"unavailable": "oracle/_ref/cuda_build/CG_cuda_ops.so not built (python oracle/build_ref_cuda.py --ref <checkout>)"}
    if wl["depthwise"]:
        return {"unavailable": "the reference has no channel-wise product (its 'mst' mode keeps the full channel product)"}
    if wl["front"] == "fast":
        wl = dict(wl, front="flat")   # the fast front end is a gather in front of the same layers; feed them directly
    taus = layer_taus(wl)
    llls = pair_list(wl)
    works = [layer_work(wl["lmax"], taus[i], taus[i + 1], llls) for i in range(wl["layers"])]
    n_ff = max(w["n_FF"] for w in works)
    B = batch
    note = None
    if 2 * B * n_ff >= 2 ** 31:
        B = max(1, (2 ** 31 - 1) // (2 * n_ff))
        note = f"batch reduced from {batch} to {B}: the reference indexes 2*B*N_FF with 32-bit integers (cudaCG_sparse.cu:17)"
    train = wl["kind"] == "train"
    keep = sum(w["n_FF"] for w in works) if train else n_ff
    free = torch.cuda.mem_get_info(dev)[0]
    if 8 * B * keep * (3 if train else 1.5) > 0.8 * free:
        return {"unavailable": f"the reference materialises the product: {8 * B * keep / 2**30:.1f} GiB at batch {B} does not fit"}
    try:
        cnn = refdrv.RefNetwork(wl["lmax"], taus, llls, dev, norm=True, seed=3)
        net = Net(cnn, wl, dev).train() if train else cnn.eval()
        params = [p for p in net.parameters() if p.requires_grad]
        opt = torch.optim.SGD(params, lr=1e-3) if wl["optimizer"] == "sgd" else None
        x, y = synth_batch(wl, 77, B)
        x, y = torch.tensor(x, device=dev), torch.tensor(y, device=dev)
        loss_fn = torch.nn.NLLLoss()

        def step():
            if not train:
                with torch.no_grad():
                    return net(x)
            for p in params:
                p.grad = None
            loss_fn(net(x), y).backward()
            if opt is not None:
                opt.step()

        step()
        torch.cuda.synchronize()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        for _ in range(steps):
            step()
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b) / steps
    except Exception as e:   # noqa: BLE001
        return {"unavailable": f"reference kernels failed: {type(e).__name__}: {e}"}
    out = {"ms_per_step": round(ms, 3), "value": round(B / (ms / 1e3), 2), "unit": "samples/s", "batch": B, "steps": steps,
           "what": "the workload's layers through the reference extension's six functions (sparse_forward, FN_WMM_forward, "
                   "FN_WMM_backward, sparse_backward; CGNet/cudaCG/cudaCG_all.cpp:39-205) in the order its modules call them, "
                   "same head, warm caches"}
    if note:
        out["note"] = note
    return out


def measure(args, wl_name, wl, dev, rank, world, batch, steps, warmup, scaling, want_kernels=True, want_ref_cuda=True,
            want_cpu=True):
    from cgnet_b200 import _lib
    lib = _lib.load()
    run = Runner(wl_name, wl, dev, rank, world, batch)
    sampler = ClockSampler(dev.index)
    if rank == 0:
        sampler.start()
    run.warm(max(warmup, 3))

    t_begin = time.time()
    lib.cgb200_launch_count(1)
    total_ms = run.timed(steps, e2e=False)
    launches = int(lib.cgb200_launch_count(0))
    e2e_ms = run.timed(steps, e2e=True)
    sampler.window = (t_begin, time.time())
    clocks = sampler.stop() if rank == 0 else None
    run.check_plans()

    kernels = {}
    if want_kernels:
        # per-kernel device time, separate instrumented pass over the same steps (events around every launch)
        nk = lib.cgb200_kernel_count()
        ms = (_lib.ctypes.c_double * nk)()
        cnt = (_lib.ctypes.c_int64 * nk)()
        lib.cgb200_timing_enable(1)
        lib.cgb200_timing_read(ms, cnt, 1)
        run.barrier()
        k_steps = min(steps, 10)
        for i in range(k_steps):
            run.flush.fill_(i & 0xFF)
            run.step(*run.dev_batches[i % run.n_batches])
        run.barrier()
        _lib.check(lib.cgb200_timing_read(ms, cnt, 1), "cgb200_timing_read")
        lib.cgb200_timing_enable(0)
        kernels = {lib.cgb200_kernel_name(k).decode(): {"launches": int(cnt[k]), "ms_total": float(ms[k]),
                                                        "us_per_launch": 1e3 * float(ms[k]) / max(int(cnt[k]), 1)}
                   for k in range(nk) if cnt[k] > 0}
    h2d = run.h2d_bytes()
    train = run.train
    del run
    torch.cuda.empty_cache()
    if rank != 0:
        return None

    peaks = {}
    try:
        peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
    except OSError:
        pass
    hbm_peak = float(peaks.get("hbm_gbs", 6650.0))
    tc_peak = float(peaks.get("bf16_tflops", 1590.0))
    peak_src = "measured (MEASURED_PEAKS.json)" if peaks else "fallback"

    # dominant kernel and its algorithmic work per launch
    B = batch
    taus = layer_taus(wl)
    llls = pair_list(wl)
    works = [layer_work(wl["lmax"], taus[i], taus[i + 1], llls, wl["depthwise"]) for i in range(wl["layers"])]
    # dominant kernel: the one with the most device time among those that do the layer's arithmetic (the layout,
    # packing and partial-sum kernels around them carry no algorithmic flops of their own)
    work_kernels = {k: v for k, v in kernels.items() if k.startswith("fused_") and not k.endswith("_reduce")}
    top = max(work_kernels, key=lambda k: work_kernels[k]["ms_total"]) if work_kernels else None
    roof = None
    if top is not None:
        kworks = works
        if top.startswith("fused_grad_f") and train and len(works) > 1:
            kworks = works[1:]    # the network's first layer needs no input gradient: that kernel runs for layers 1..
        # every fused kernel launches once per layer per step; average the per-layer work over the layers.  Algorithmic
        # work only: the product regenerated by the backward kernels is recomputation, not counted.
        if top.startswith("fused_fwd"):
            flops = [w["cg_flops"] + w["mix_flops"] for w in kworks]
        elif top == "fused_stats":
            flops = [w["cg_flops"] for w in kworks]
        elif top.startswith("fused_grad_w"):
            flops = [w["mix_flops"] for w in kworks]                      # gW = gO^T conj(FF): one mixing-sized contraction
        elif top.startswith("fused_grad_f") and "grad_mid_tensor" in kernels:
            flops = [2 * w["cg_flops"] for w in kworks]                   # the product's two operand roles; gFF comes from grad_mid_tensor
        elif top.startswith("fused_grad_f"):
            flops = [2 * w["cg_flops"] + w["mix_flops"] for w in kworks]  # gFF (mixing-sized) + the product's two operand roles
        else:
            flops = [0 for _ in kworks]
        byts = [8 * B * (w["n_F"] + w["n_O"]) + 8 * w["w_len"] + 4 * w["sum_tff"] + 4 * w["cg_len"] for w in kworks]
        dur_s = kernels[top]["us_per_launch"] * 1e-6
        flop_per_launch = B * sum(flops) / len(kworks)
        achieved_tf = flop_per_launch / dur_s / 1e12 if dur_s > 0 else 0.0
        sm_mhz = (clocks or {}).get("sm_mhz") or peaks.get("sm_max_mhz", 1965.0)
        simt_peak_tf = 148 * 128 * 2 * float(sm_mhz) * 1e6 / 1e12
        on_tensor = top.endswith("_tensor")
        roof = {"kernel": top, "bound": "tensor" if on_tensor else "cuda_core_fp32",
                "achieved": round(achieved_tf, 3), "peak": tc_peak if on_tensor else round(simt_peak_tf, 1), "unit": "TFLOP/s",
                "frac": round(achieved_tf / (tc_peak if on_tensor else simt_peak_tf), 5),
                "traffic": NCU_TRAFFIC.get((wl_name, top)),
                "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum of one captured launch; see profiles/)",
                "peak_source": (peak_src + ", dense bf16 burst") if on_tensor else "148 SMs x 128 fp32 lanes x 2 x SM clock sampled during the run",
                "algorithmic_flop_per_launch": flop_per_launch,
                "algorithmic_bytes_per_launch": sum(byts) / len(kworks),
                "frac_of_tensor_peak": round(achieved_tf / tc_peak, 5),
                "frac_of_hbm_peak": round(sum(byts) / len(kworks) / dur_s / 1e9 / hbm_peak, 5) if dur_s > 0 else None,
                "frac_of_cuda_core_fp32_peak": round(achieved_tf / simt_peak_tf, 4),
                "note": "the CG product is generated on the fp32 CUDA cores in every kernel (the tensor-core kernels move the "
                        "mixing-sized contractions to tcgen05), so a kernel that is not a *_tensor kernel is held to the fp32 "
                        "SIMT peak; its fractions of the measured tensor and HBM peaks are given beside it"}

    ms_step = total_ms / steps
    n_samples = world * B if scaling == "weak" else args.global_batch
    metric = METRIC_TRAIN if train else METRIC_LAYER if wl["kind"] == "layer_infer" else METRIC_INFER
    out = {
        "metric": metric, "value": round(n_samples / (ms_step / 1e3), 1),
        "unit": "samples/s", "n_gpus": world, "steps": steps, "warmup": max(warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "describe": wl["describe"], "per_gpu_batch": B, "global_batch": n_samples,
                   "l2": "flushed between timed steps (256 MB write, outside the timed intervals)",
                   "parallelism": f"dp{world}", "pairs": wl["pairs"], "depthwise": wl["depthwise"],
                   "fragment_norm": "training mode (statistics updated every step)" if train else "inference (stored statistics)"},
        "e2e": {"value": round(n_samples / (e2e_ms / steps / 1e3), 1), "unit": "samples/s",
                "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4, "ms_per_step": round(e2e_ms / steps, 4)},
        "gpu_launches": launches, "gpu_launches_per_step": launches / steps,
        "clocks": clocks, "roofline": roof, "kernels": kernels,
    }
    if want_ref_cuda:
        ref = time_reference_cuda(wl, dev, B, steps=3 if ms_step > 5 else 10)
        if "ms_per_step" in ref:
            ref["speedup"] = round((B / (ms_step / 1e3)) / ref["value"], 2)   # this GPU's samples/s over the reference kernels'

        out["reference_cuda"] = ref
    if want_cpu:
        out["cpu_baseline"] = cpu_baseline(wl, sample=cpu_sample(wl), repeats=1)
    return out


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's Python layer
# ---------------------------------------------------------------------------------------------------------------
def cpu_step(wl, x, y, weights, stds_list, llls):
    """Forward (+ backward for the training workloads) on the CPU with the oracle (torch CPU ops, reference's algorithm)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cg_oracle as o
    lmax = wl["lmax"]
    taus = layer_taus(wl)
    B = x.shape[0]
    if wl["kind"] != "train":
        with torch.no_grad():
            fs = o.split_fragments(x, taus[0])
            for i in range(wl["layers"]):
                if wl["depthwise"]:
                    fs, _ = o.cgbn_layer(fs, taus[i], taus[i + 1], lmax, llls, weights[i], stds=stds_list[i], depthwise=True)
                else:
                    fs = o.twin_forward(fs, taus[i], taus[i + 1], lmax, llls, weights[i], stds=stds_list[i])
        return float(fs[0].sum().item())
    Ws = [w.clone().requires_grad_(True) for w in weights]
    fs = o.split_fragments(x, taus[0])
    emb = [fs[0].reshape(B, -1)]
    for i in range(wl["layers"]):
        fs, _ = o.twin_forward(fs, taus[i], taus[i + 1], lmax, llls, Ws[i], stds=stds_list[i], training=True, cnt=1.0)
        emb.append(fs[0].reshape(B, -1))
    e = torch.cat(emb, 1)
    head = cpu_step.head
    out = torch.log_softmax(head[2](torch.relu(head[1](head[0](e)))), dim=1)
    loss = torch.nn.functional.nll_loss(out, y)
    loss.backward()
    return float(loss.item())


def cpu_sample(wl):
    """Samples per CPU step for the reported baseline: a few seconds of host work, from the workload's flop count."""
    taus = layer_taus(wl)
    llls = pair_list(wl)
    flops = sum(sum(layer_work(wl["lmax"], taus[i], taus[i + 1], llls, wl["depthwise"])[k] for k in ("cg_flops", "mix_flops"))
                for i in range(wl["layers"]))
    flops *= 3 if wl["kind"] == "train" else 1
    return int(max(1, min(4, 40e9 // max(flops, 1))))


def cpu_baseline(wl, sample, repeats):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cg_oracle as o
    torch.set_num_threads(os.cpu_count() or 1)
    lmax = wl["lmax"]
    flat = dict(wl, front="flat")
    taus = layer_taus(wl)
    llls = pair_list(wl)
    rng = np.random.RandomState(7)
    weights, stds_list = [], []
    for i in range(wl["layers"]):
        if wl["depthwise"]:
            t_ff = np.zeros(lmax + 1, dtype=np.int64)
            for l, l1, l2 in o.decode_triples(lmax, llls):
                t_ff[l] += taus[i][l1]
        else:
            t_ff, _ = o.tau_ff_and_offsets(lmax, taus[i], llls)
        weights.append(torch.tensor(0.05 * rng.rand(int((t_ff * np.asarray(taus[i + 1])).sum()), 2), dtype=torch.float32))
        stds_list.append((0.5 + rng.rand(int(t_ff.sum()))).astype(np.float32))
    n_emb = 2 * sum(t[0] for t in taus)
    torch.manual_seed(7)
    if wl["kind"] == "train":
        cpu_step.head = (torch.nn.BatchNorm1d(n_emb), torch.nn.Linear(n_emb, wl["hidden"]), torch.nn.Linear(wl["hidden"], wl["classes"]))
    x, y = synth_batch(flat, 99, batch=sample)
    x, y = torch.tensor(x), torch.tensor(y)
    t0 = time.perf_counter()
    cpu_step(wl, x, y, weights, stds_list, llls)             # warm-up (also fills the oracle's CG cache)
    warm = time.perf_counter() - t0
    t0 = time.perf_counter()
    for _ in range(repeats):
        cpu_step(wl, x, y, weights, stds_list, llls)
    dt = (time.perf_counter() - t0) / repeats
    return {"value": round(sample / dt, 3), "unit": "samples/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample} of the workload's {wl['batch']} samples per step, {repeats} timed step(s) after one warm-up; "
                      "oracle/cg_oracle.py (the reference's per-triple Kronecker + bmm algorithm) + torch autograd on the host CPU",
            "seconds_per_step": round(dt, 3), "warmup_seconds": round(warm, 3)}


def run_reference(args, wl_name, wl):
    """The CPU arm: the restated Python layer on the workload's own batch where a step of it stays within about 25 s of
    host time, otherwise on the largest sample that does (stated in `config`)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    probe = cpu_baseline(wl, sample=cpu_sample(wl), repeats=1)
    rate = probe["value"]
    sample = int(max(1, min(wl["batch"], rate * 25)))
    steps = max(1, min(args.steps, 3))
    cpu = cpu_baseline(wl, sample=sample, repeats=steps) if sample != cpu_sample(wl) else probe
    metric = METRIC_TRAIN if wl["kind"] == "train" else METRIC_LAYER if wl["kind"] == "layer_infer" else METRIC_INFER
    return {
        "impl": "reference", "metric": metric, "value": cpu["value"],
        "unit": "samples/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": 1,
        "ms_per_step": round(1e3 * cpu["seconds_per_step"], 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "describe": wl["describe"], "per_step_sample": sample, "workload_batch": wl["batch"],
                   "note": "CPU restatement of the reference's Python layer (CGNet/CG_layers_python.py) on the host cores; "
                           "the reference's own Python files need a GPU even for that path (CG_layers_python.py:177,242) and "
                           "cannot travel to the GPU box; its CUDA kernels are timed as `reference_cuda` in the default arm's line"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def run_ours(args, wl_name, wl):
    import torch.distributed as dist
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device for the default arm (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    scaling = "weak"
    batch = wl["batch"]
    if args.global_batch:
        from cgnet_b200.dp import shard_batch
        sl = shard_batch(args.global_batch, rank, world)
        batch, scaling = sl.stop - sl.start, "strong"
        if batch == 0:
            raise RuntimeError("--global-batch smaller than the number of ranks")
    out = measure(args, wl_name, wl, dev, rank, world, batch, args.steps, args.warmup, scaling,
                  want_ref_cuda=not args.no_reference_cuda and world == 1, want_cpu=not args.no_cpu_baseline and world == 1)
    if wl_name == "cgnet5_lmax10" and not args.no_lmax20 and not args.global_batch:
        # the other degree the headline metric names, in the same record: a short run of the lmax-20 network (inference,
        # no exchange between ranks: every rank runs a replica on its own batch)
        extra = {}
        for name in ("mst_lmax20_tau32", "mst_lmax20_tau32_depthwise"):
            w2 = WORKLOADS[name]
            r = measure(args, name, w2, dev, rank, world, w2["batch"], steps=5, warmup=3, scaling="weak", want_kernels=True,
                        want_ref_cuda=False, want_cpu=False)
            if r is not None:
                extra[name] = {k: r[k] for k in ("metric", "value", "unit", "ms_per_step", "steps", "config", "e2e", "roofline", "clocks")}
                extra[name]["kernels"] = {k: round(v["us_per_launch"], 1) for k, v in r["kernels"].items()}
        if out is not None:
            out["lmax20"] = extra
    if world > 1:
        dist.destroy_process_group()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cgnet5_lmax10", choices=sorted(WORKLOADS))
    ap.add_argument("--global-batch", type=int, default=0, help="split this many samples over the ranks (strong scaling)")
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the reference's CUDA kernels")
    ap.add_argument("--no-lmax20", action="store_true", help="skip the short lmax-20 runs appended to the default workload's line")
    ap.add_argument("--list", action="store_true")
    args = ap.parse_args()
    if args.list:
        for k in sorted(WORKLOADS):
            print(f"{k:32s} {WORKLOADS[k]['describe']}")
        return
    wl = WORKLOADS[args.workload]
    # stdout carries exactly one JSON line: anything a library prints there meanwhile (NCCL's version banner, ...) is
    # sent to stderr
    real_stdout = os.dup(1)
    os.dup2(2, 1)
    out = run_reference(args, args.workload, wl) if args.impl == "reference" else run_ours(args, args.workload, wl)
    sys.stdout.flush()
    os.dup2(real_stdout, 1)
    if out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
