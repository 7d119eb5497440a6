#!/usr/bin/env python
"""Benchmark of the CG-layer hot path:  samples/s of a CG network training step (forward + backward).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload cgnet5_lmax10]

Workloads (synthetic, seeded; shapes of BASELINE.json's configs):
  cgnet5_lmax10   5 CG layers, lmax 10, tau 1 -> 5, full pair list, fragment norm in training mode, skip-concatenated
                  l=0 invariants -> BatchNorm1d -> Linear(52,256) -> ReLU -> Linear(256,10) -> log-softmax -> NLL;
                  batch 100 per GPU; input coefficient (l, m) ~ complex N(0, 1/(2l+1)).  Forward + backward.
  layer_lmax5     one CG layer, lmax 5, tau 8, batch 32 (the reference's CPU-runnable case), forward + backward.

One JSON line is printed by rank 0.  `value` is timed with CUDA events around each step with the inputs already in
HBM, the L2 flushed (a 256 MB write) between steps and outside the timed intervals; `e2e` repeats the measurement through
the public module call with the step's input copied from pinned host memory and the loss read back to the host inside
the timed interval.  With N > 1 every rank processes its own batch (weak scaling) and the step ends with the NCCL
all-reduce of all gradients; times are the maximum over ranks.

`--impl reference` times the CPU restatement of the reference's own Python layer (oracle/cg_oracle.py, torch CPU ops
with all host threads) on a bounded sample of the same workload.
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
METRIC_INFER = "fused CG layer samples/sec (inference forward)"

WORKLOADS = {
    "cgnet5_lmax10": dict(lmax=10, tau_in=1, tau=5, layers=5, batch=100, hidden=256, classes=10,
                          describe="5-layer CGNet lmax=10 tau=5 batch=100 fwd+bwd (BASELINE configs[1])"),
    "layer_lmax5": dict(lmax=5, tau_in=8, tau=8, layers=1, batch=32, hidden=256, classes=10,
                        describe="single CG layer lmax=5 tau=8 batch=32 fwd+bwd (BASELINE configs[0] shape)"),
    "cgnet2_lmax14_tau16": dict(lmax=14, tau_in=16, tau=16, layers=2, batch=64, hidden=256, classes=10,
                                describe="2-layer CGNet lmax=14 tau=16 batch=64 fwd+bwd (layer shape of BASELINE configs[2]; "
                                         "tensor-core forward and weight gradient)"),
    # single fused layer, inference forward only (BASELINE configs[4], the sweep's points that fit a quick run)
    "fused_layer_lmax10_tau16": dict(kind="layer_infer", lmax=10, tau_in=16, tau=16, layers=1, batch=256, classes=10, hidden=0,
                                     describe="one fused CG layer lmax=10 tau=16 batch=256, inference forward (BASELINE configs[4])"),
    "fused_layer_lmax10_tau32": dict(kind="layer_infer", lmax=10, tau_in=32, tau=32, layers=1, batch=128, classes=10, hidden=0,
                                     describe="one fused CG layer lmax=10 tau=32 batch=128, inference forward (BASELINE configs[4])"),
    "fused_layer_lmax10_tau64": dict(kind="layer_infer", lmax=10, tau_in=64, tau=64, layers=1, batch=64, classes=10, hidden=0,
                                     describe="one fused CG layer lmax=10 tau=64 batch=64, inference forward (BASELINE configs[4])"),
}


def synth_batch(wl, seed, batch=None):
    """Seeded stand-in for spherical-harmonic coefficients of a band-limited function: variance 1/(2l+1) per degree."""
    B = batch or wl["batch"]
    rng = np.random.RandomState(seed)
    parts = []
    for l in range(wl["lmax"] + 1):
        parts.append(rng.randn(B, wl["tau_in"] * (2 * l + 1), 2) / np.sqrt(2.0 * (2 * l + 1)))
    x = np.concatenate(parts, axis=1).astype(np.float32)
    y = rng.randint(0, wl["classes"], size=B).astype(np.int64)
    return x, y


def layer_taus(wl):
    L1 = wl["lmax"] + 1
    return [[wl["tau_in"]] * L1] + [[wl["tau"]] * L1 for _ in range(wl["layers"])]


# ---------------------------------------------------------------------------------------------------------------
# algorithmic work per sample (forward), from the shapes alone
# ---------------------------------------------------------------------------------------------------------------
def layer_work(lmax, taus, tau_out):
    from cgnet_b200 import CGutils
    llls = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(CGutils.SparseLtuples.compute_default_ltuples(lmax))[0]
    cg_flops = 0
    t_ff = np.zeros(lmax + 1, dtype=np.int64)
    cg_len = 0
    for l, l1, l2 in CGutils.SparseLtuples.get_iter(lmax, llls):
        nnz = sum(1 for m in range(-l, l + 1) for m2 in range(-l2, l2 + 1) if abs(m - m2) <= l1)
        cg_flops += 8 * taus[l1] * taus[l2] * nnz
        t_ff[l] += taus[l1] * taus[l2]
        cg_len += (2 * l + 1) * (2 * l2 + 1)
    n = 2 * np.arange(lmax + 1) + 1
    mix_flops = int(8 * (t_ff * np.asarray(tau_out) * n).sum())
    return dict(cg_flops=int(cg_flops), mix_flops=mix_flops, n_F=int((np.asarray(taus) * n).sum()),
                n_O=int((np.asarray(tau_out) * n).sum()), n_FF=int((t_ff * n).sum()), w_len=int((t_ff * np.asarray(tau_out)).sum()),
                sum_tff=int(t_ff.sum()), cg_len=int(cg_len))


# ---------------------------------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------------------------------
class Net(torch.nn.Module):
    """The reference's MNIST classifier shape (MNIST/model.py:28-67) on top of SphericalCNN, dropout left out."""

    def __init__(self, wl, device):
        super().__init__()
        from cgnet_b200 import SphericalCNN
        self.cnn = SphericalCNN(wl["lmax"], layer_taus(wl), norm=True, skipconn=True, device=device)
        n = self.cnn.output_length
        self.bm1 = torch.nn.BatchNorm1d(n)
        self.fc = torch.nn.Linear(n, wl["hidden"])
        self.final = torch.nn.Linear(wl["hidden"], wl["classes"])
        self.to(device)

    def forward(self, x):
        x = self.bm1(self.cnn(x))
        x = torch.relu(self.fc(x))
        return torch.log_softmax(self.final(x), dim=1)


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


def run_ours(args, wl_name, wl):
    import torch.distributed as dist
    from cgnet_b200 import _lib
    from cgnet_b200.dp import GradientAverager, broadcast_parameters

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device for the default arm (there is no CPU fallback)")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    lib = _lib.load()

    torch.manual_seed(1234)
    np.random.seed(1234)
    infer = wl.get("kind") == "layer_infer"
    if infer:
        from cgnet_b200 import CGBN_cuda
        L1 = wl["lmax"] + 1
        net = CGBN_cuda(wl["lmax"], [wl["tau_in"]] * L1, [wl["tau"]] * L1, batchnorm=True, device=dev)
        net.eval()
    else:
        net = Net(wl, dev)
        net.train()
    if world > 1:
        broadcast_parameters(net)
    params = [p for p in net.parameters() if p.requires_grad]
    # the network's gradients are 1.5 MB: one bucket, one all-reduce on the compute stream after the backward pass
    # (measured on two GPUs: +0.035 ms per step; per-layer buckets started inside the backward pass cost +0.10 ms,
    # because each collective takes SMs from the persistent backward kernels)
    averager = GradientAverager(params, average=True, bucket_bytes=64 << 20, overlap=False) if world > 1 and not infer else None
    B = wl["batch"]
    n_batches = 4
    host = [synth_batch(wl, 100 + rank * n_batches + i) for i in range(n_batches)]
    dev_batches = [(torch.tensor(x, device=dev), torch.tensor(y, device=dev)) for x, y in host]
    pinned = [(torch.tensor(x).pin_memory(), torch.tensor(y).pin_memory()) for x, y in host]
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    loss_fn = torch.nn.NLLLoss()

    def step(x, y):
        if infer:
            with torch.no_grad():
                return net(x, straight_output=True)[:, :8].sum()   # a small read-back value for the end-to-end pass
        for p in params:
            p.grad = None
        loss = loss_fn(net(x), y)
        loss.backward()
        if averager is not None:
            averager.finish()
        return loss

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(n_steps, e2e):
        """Sum of per-step device times (ms); L2 flush between steps, outside the timed intervals."""
        ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n_steps)]
        barrier()
        for i in range(n_steps):
            flush.fill_(i & 0xFF)
            ev[i][0].record()
            if e2e:
                xh, yh = pinned[i % n_batches]
                x = xh.to(dev, non_blocking=True)
                y = yh.to(dev, non_blocking=True)
                loss = step(x, y)
                loss.item()               # device -> host read of the step's result, inside the timed interval
            else:
                x, y = dev_batches[i % n_batches]
                step(x, y)
            ev[i][1].record()
        barrier()
        total = sum(a.elapsed_time(b) for a, b in ev)
        t = torch.tensor([total], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for i in range(max(args.warmup, 3)):
        step(*dev_batches[i % n_batches])
    barrier()

    t_begin = time.time()
    lib.cgb200_launch_count(1)
    total_ms = timed(args.steps, e2e=False)
    launches = int(lib.cgb200_launch_count(0))
    e2e_ms = timed(args.steps, e2e=True)
    sampler.window = (t_begin, time.time())
    clocks = sampler.stop() if rank == 0 else None

    # per-kernel device time, separate instrumented pass over the same steps (events around every launch)
    nk = lib.cgb200_kernel_count()
    ms = (_lib.ctypes.c_double * nk)()
    cnt = (_lib.ctypes.c_int64 * nk)()
    lib.cgb200_timing_enable(1)
    lib.cgb200_timing_read(ms, cnt, 1)
    barrier()
    for i in range(args.steps):
        flush.fill_(i & 0xFF)
        step(*dev_batches[i % n_batches])
    barrier()
    _lib.check(lib.cgb200_timing_read(ms, cnt, 1), "cgb200_timing_read")
    lib.cgb200_timing_enable(0)
    kernels = {lib.cgb200_kernel_name(k).decode(): {"launches": int(cnt[k]), "ms_total": float(ms[k]),
                                                    "us_per_launch": 1e3 * float(ms[k]) / max(int(cnt[k]), 1)}
               for k in range(nk) if cnt[k] > 0}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
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
    taus = layer_taus(wl)
    works = [layer_work(wl["lmax"], taus[i], taus[i + 1]) for i in range(wl["layers"])]
    top = max(kernels, key=lambda k: kernels[k]["ms_total"]) if kernels else None
    roof = None
    if top is not None:
        if top == "fused_grad_f" and not infer and len(works) > 1:
            works = works[1:]     # the network's first layer needs no input gradient: that kernel runs for layers 1..
        # every fused kernel launches once per layer per step; average the per-layer work over the layers
        if top in ("fused_fwd", "fused_fwd_tensor"):
            flops = [w["cg_flops"] + w["mix_flops"] for w in works]
        elif top == "fused_stats":
            flops = [w["cg_flops"] for w in works]
        elif top in ("fused_grad_w", "fused_grad_f"):
            # weight gradient: regenerate the product + one mixing-sized contraction; input gradient: one
            # mixing-sized contraction + the product's two operand roles
            flops = [w["cg_flops"] + w["mix_flops"] if top == "fused_grad_w" else 2 * w["cg_flops"] + w["mix_flops"] for w in works]
        else:
            flops = [0 for _ in works]
        byts = [8 * B * (w["n_F"] + w["n_O"]) + 8 * w["w_len"] + 4 * w["sum_tff"] + 4 * w["cg_len"] for w in works]
        dur_s = kernels[top]["us_per_launch"] * 1e-6
        flop_per_launch = B * sum(flops) / len(works)
        achieved_tf = flop_per_launch / dur_s / 1e12 if dur_s > 0 else 0.0
        sm_mhz = (clocks or {}).get("sm_mhz") or peaks.get("sm_max_mhz", 1965.0)
        simt_peak_tf = 148 * 128 * 2 * float(sm_mhz) * 1e6 / 1e12
        roof = {"kernel": top, "bound": "tensor", "achieved": round(achieved_tf, 3), "peak": tc_peak, "unit": "TFLOP/s",
                "frac": round(achieved_tf / tc_peak, 5), "traffic": NCU_TRAFFIC.get((wl_name, top)),
                "traffic_unit": "bytes per launch (ncu dram__bytes_read.sum + dram__bytes_write.sum of one captured launch; see profiles/)",
                "peak_source": peak_src,
                "algorithmic_flop_per_launch": flop_per_launch,
                "algorithmic_bytes_per_launch": sum(byts) / len(works),
                "hbm_frac_of_algorithmic_bytes": round(sum(byts) / len(works) / dur_s / 1e9 / hbm_peak, 5) if dur_s > 0 else None,
                "cuda_core_fp32": {"achieved": round(achieved_tf, 3), "peak": round(simt_peak_tf, 1), "unit": "TFLOP/s",
                                   "frac": round(achieved_tf / simt_peak_tf, 4),
                                   "note": "CG-product generation runs on the fp32 CUDA cores in every kernel (the tensor-core forward "
                                           "moves only the mixing to tcgen05); peak = 148 SMs x 128 lanes x 2 x sampled SM clock"}}

    cpu = None if args.no_cpu_baseline else cpu_baseline(wl, sample=4, repeats=1)
    ms_step = total_ms / args.steps
    out = {
        "metric": METRIC_INFER if infer else METRIC_TRAIN, "value": round(world * B / (ms_step / 1e3), 1),
        "unit": "samples/s", "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": round(ms_step, 4),
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "describe": wl["describe"], "per_gpu_batch": B, "global_batch": B * world,
                   "l2": "flushed between timed steps (256 MB write, outside the timed intervals)",
                   "parallelism": f"dp{world}",
                   "fragment_norm": "inference (stored statistics)" if infer else "training mode (statistics updated every step)"},
        "e2e": {"value": round(world * B / (e2e_ms / args.steps / 1e3), 1), "unit": "samples/s",
                "h2d_bytes_per_step": int(pinned[0][0].numel() * 4 + pinned[0][1].numel() * 8), "d2h_bytes_per_step": 4,
                "ms_per_step": round(e2e_ms / args.steps, 4)},
        "gpu_launches": launches, "gpu_launches_per_step": launches / args.steps,
        "clocks": clocks, "roofline": roof, "kernels": kernels, "cpu_baseline": cpu,
    }
    if world > 1:
        dist.destroy_process_group()
    return out


# ---------------------------------------------------------------------------------------------------------------
# CPU arm: the oracle's restatement of the reference's Python layer
# ---------------------------------------------------------------------------------------------------------------
def cpu_step(wl, x, y, weights, stds_list):
    """Forward + backward of the workload on the CPU with the oracle (torch CPU ops, reference's algorithm)."""
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cg_oracle as o
    lmax = wl["lmax"]
    taus = layer_taus(wl)
    llls, _ = o.encode_sorted(o.default_ltuples(lmax))
    B = x.shape[0]
    if wl.get("kind") == "layer_infer":
        with torch.no_grad():
            out = o.twin_forward(o.split_fragments(x, taus[0]), taus[0], taus[1], lmax, llls, weights[0], stds=stds_list[0])
        return float(out[0].sum().item())
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


def cpu_baseline(wl, sample, repeats):
    sys.path.insert(0, os.path.join(ROOT, "oracle"))
    import cg_oracle as o
    torch.set_num_threads(os.cpu_count() or 1)
    lmax = wl["lmax"]
    taus = layer_taus(wl)
    llls, _ = o.encode_sorted(o.default_ltuples(lmax))
    rng = np.random.RandomState(7)
    weights, stds_list = [], []
    for i in range(wl["layers"]):
        t_ff, _ = o.tau_ff_and_offsets(lmax, taus[i], llls)
        weights.append(torch.tensor(0.05 * rng.rand(int((t_ff * np.asarray(taus[i + 1])).sum()), 2), dtype=torch.float32))
        stds_list.append((0.5 + rng.rand(int(t_ff.sum()))).astype(np.float32))
    n_emb = 2 * sum(t[0] for t in taus)
    torch.manual_seed(7)
    cpu_step.head = (torch.nn.BatchNorm1d(n_emb), torch.nn.Linear(n_emb, wl["hidden"]), torch.nn.Linear(wl["hidden"], wl["classes"]))
    x, y = synth_batch(wl, 99, batch=sample)
    x, y = torch.tensor(x), torch.tensor(y)
    cpu_step(wl, x, y, weights, stds_list)             # warm-up (also fills the oracle's CG cache)
    t0 = time.perf_counter()
    for _ in range(repeats):
        cpu_step(wl, x, y, weights, stds_list)
    dt = (time.perf_counter() - t0) / repeats
    return {"value": round(sample / dt, 3), "unit": "samples/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"{sample} of the workload's {wl['batch']} samples per step, {repeats} timed step(s) after one warm-up; "
                      "oracle/cg_oracle.py twin_forward + torch autograd on the host CPU",
            "seconds_per_step": round(dt, 3)}


def run_reference(args, wl_name, wl):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    sample = 8
    steps = max(1, min(args.steps, 3))
    cpu = cpu_baseline(wl, sample=sample, repeats=steps)
    return {
        "impl": "reference", "metric": METRIC_INFER if wl.get("kind") == "layer_infer" else METRIC_TRAIN, "value": cpu["value"],
        "unit": "samples/s", "n_gpus": int(os.environ.get("WORLD_SIZE", "1")), "steps": steps, "warmup": 1,
        "ms_per_step": round(1e3 * cpu["seconds_per_step"], 2), "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": wl_name, "describe": wl["describe"], "per_step_sample": sample,
                   "note": "CPU restatement of the reference's Python layer (CGNet/CG_layers_python.py) on the host cores; "
                           "the reference's own files cannot travel to the GPU box, and its CUDA extension is not a CPU path"},
        "cpu_baseline": cpu,
        "e2e": {"value": cpu["value"], "unit": "samples/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=30)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="cgnet5_lmax10", choices=sorted(WORKLOADS))
    ap.add_argument("--no-cpu-baseline", action="store_true", help="skip the CPU leg (profiling runs)")
    args = ap.parse_args()
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
