"""Shared helpers of the parity tests: seeded inputs, per-fragment error, oracle runs."""
import numpy as np
import torch

import cg_oracle as o

TOL = 1e-4   # relative Frobenius error per fragment, fp32: the bar the parity tests hold the CUDA path to


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b)
    return float(np.linalg.norm(a - b) / d) if d > 0 else float(np.linalg.norm(a))


def assert_fragments_close(got, want, taus, what, tol=TOL):
    """got/want: flat (B, N, 2) arrays; compared fragment by fragment."""
    got = np.asarray(got)
    want = np.asarray(want)
    assert got.shape == want.shape, (what, got.shape, want.shape)
    off = 0
    for l, t in enumerate(taus):
        n = int(t) * (2 * l + 1)
        if n:
            err = rel_fro(got[:, off:off + n], want[:, off:off + n])
            assert err < tol, f"{what}: fragment l={l} relative Frobenius error {err:.3e} >= {tol}"
        off += n
    assert off == got.shape[1]


def assert_weights_close(got, want, t_ff, tau_out, what, tol=TOL):
    off = 0
    for l in range(len(t_ff)):
        n = int(t_ff[l]) * int(tau_out[l])
        if n:
            err = rel_fro(got[off:off + n], want[off:off + n])
            assert err < tol, f"{what}: degree l={l} relative Frobenius error {err:.3e} >= {tol}"
        off += n


def ltuples(mode, lmax):
    return {"default": o.default_ltuples, "mst": o.mst_ltuples, "debug": o.debug_ltuples}[mode](lmax)


def make_case(taus, tau_out, B, mode="default", seed=0, depthwise=False, scale=1.0):
    """Seeded inputs for one layer plus everything the oracle derives from the shapes."""
    lmax = len(taus) - 1
    llls, _ = o.encode_sorted(ltuples(mode, lmax) if isinstance(mode, str) else mode)
    if depthwise:
        t_ff = np.zeros(lmax + 1, dtype=np.int64)
        for l, l1, l2 in o.decode_triples(lmax, llls):
            t_ff[l] += taus[l1]
    else:
        t_ff, _ = o.tau_ff_and_offsets(lmax, taus, llls)
    rng = np.random.RandomState(seed)
    n_f = int(o.cumulative_tm(taus)[-1])
    n_o = int(o.cumulative_tm(tau_out)[-1])
    case = dict(lmax=lmax, taus=list(taus), tau_out=list(tau_out), llls=llls, t_ff=t_ff, B=B, depthwise=depthwise)
    case["F"] = (scale * rng.randn(B, n_f, 2)).astype(np.float32)
    wlen = int((t_ff * np.asarray(tau_out)).sum())
    case["W"] = (0.05 * rng.rand(wlen, 2)).astype(np.float32)
    case["stds"] = (0.25 + rng.rand(int(t_ff.sum()))).astype(np.float32)
    case["gO"] = rng.randn(B, n_o, 2).astype(np.float32)
    case["gFF"] = rng.randn(B, int(o.cumulative_tm(t_ff)[-1]), 2).astype(np.float32)
    return case


def oracle_product(case, dtype=torch.float64):
    """FF and d<FF, gFF>/dF from the oracle."""
    F = torch.tensor(case["F"], dtype=dtype, requires_grad=True)
    ff = o.join_fragments(o.cg_product(o.split_fragments(F, case["taus"]), case["taus"], case["lmax"], case["llls"],
                                       depthwise=case["depthwise"]))
    (ff * torch.tensor(case["gFF"], dtype=dtype)).sum().backward()
    return ff.detach().numpy(), F.grad.numpy()


def oracle_layer(case, bn, training=False, cnt=1.0, eps=1e-5, dtype=torch.float64):
    """O, gF, gW (for the cotangent gO) and the updated stds from the oracle.  bn: use case['stds'] or no norm."""
    F = torch.tensor(case["F"], dtype=dtype, requires_grad=True)
    W = torch.tensor(case["W"], dtype=dtype, requires_grad=True)
    out, new_stds = o.cgbn_layer(o.split_fragments(F, case["taus"]), case["taus"], case["tau_out"], case["lmax"],
                                 case["llls"], W, stds=case["stds"] if bn else None, eps=eps, cnt=cnt, training=training,
                                 depthwise=case["depthwise"])
    O = o.join_fragments(out)
    (O * torch.tensor(case["gO"], dtype=dtype)).sum().backward()
    gF = F.grad.numpy() if F.grad is not None else np.zeros_like(case["F"], dtype=np.float64)
    return O.detach().numpy(), gF, W.grad.numpy(), new_stds
