"""Generate the golden fixtures in this directory by RUNNING THE REFERENCE's own CPU code.

    python tests/golden/make_golden.py [--ref /path/to/CGNet-checkout]

Needs a checkout of zlin7/CGNet (the --ref argument) and its ``ClebschGordan`` C++ module built by
``make -C oracle ref``.  The fixtures it writes (``*.npz``, a few hundred kB in total) are committed, so the test-suite
itself never needs the checkout.

What is executed from the reference, unmodified, on the CPU:
  * ``CGNet.CGutils``: ``SparseLtuples`` (pair lists, canonical order, offsets), ``compute_MST``, ``ClebschGordanDict``,
    ``Complex_bmm``, ``reshape_out``;
  * ``CGNet.CG_layers_python``: ``CG_sparse_py`` (the CG product) and ``MyBatchNormList`` in eval mode;
  * the compiled ``ClebschGordan.precompute``;
  * torch autograd through those for the gradients.
Two import shims are needed and change no arithmetic: a stub ``ipdb`` module (a debugger the files import but never
call) and ``np.int = int`` (an alias numpy removed).

What is NOT the reference's own code, because the reference cannot run it without a GPU: the layer composition of
``CGBN_base.forward`` (its constructor allocates weights on 'cuda', ``CG_layers_python.py:242``) and the training-mode
statistics of ``MyBatchNormList.forward`` (which call ``.cuda()``, ``:177``).  Both are transcribed below, line for
line in meaning, around the reference's functions; the fixtures that depend on them are stored under keys that begin
with ``harness_``.
"""
import argparse
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))


def import_reference(ref):
    sys.modules.setdefault("ipdb", types.ModuleType("ipdb"))
    if not hasattr(np, "int"):
        np.int = int  # noqa: NPY001  (alias used at CGutils.py:125,134)
    sys.path.insert(0, os.path.join(ROOT, "oracle", "_ref"))
    sys.path.insert(0, ref)
    import CGNet.CGutils as cgu
    import CGNet.CG_layers_python as cgpy
    return cgu, cgpy


def index_fixtures(cgu):
    out = {}
    cases = [("default", 2), ("default", 4), ("default", 5), ("default", 10), ("default", 14),
             ("mst", 2), ("mst", 4), ("mst", 6), ("mst", 10), ("mst", 20), ("debug", 3), ("debug", 5)]
    for mode, L in cases:
        if mode == "default":
            lt = cgu.SparseLtuples.compute_default_ltuples(L)
        elif mode == "debug":
            lt = cgu.SparseLtuples.compute_debug_ltuples(L)
        else:
            lt = []
            for l in range(L + 1):
                l1s, l2s = cgu.compute_MST(l, L, diag=True)
                lt.append(list(zip(l1s, l2s)))
            # raw per-l pair lists, before the stable sort, flattened as (l, l1, l2) rows
            out[f"{mode}_{L}_rawpairs"] = np.array([(l, a, b) for l in range(L + 1) for a, b in lt[l]], dtype=np.int32)
        llls, table = cgu.SparseLtuples.sparse_rep_ltuples_sorted(lt)
        out[f"{mode}_{L}_llls"] = np.asarray(llls, dtype=np.int64)
        out[f"{mode}_{L}_l_l1_offsets"] = np.asarray(table, dtype=np.int64)
        out[f"{mode}_{L}_cg_offsets"] = np.asarray(cgu.SparseLtuples.cal_CG_offsets(L, llls), dtype=np.int64)
        assert cgu.SparseLtuples.get_CG_length(L, llls) == out[f"{mode}_{L}_cg_offsets"][-1]
        for tag, taus in (("ones", [1] * (L + 1)), ("ramp", [1 + (3 * l) % 4 for l in range(L + 1)])):
            # CG_sparse_py.cal_new_tau_and_offsets == CG_woFilter_cuda.cal_new_tau_and_offsets, minus the constructor
            t_ff = np.zeros(L + 1, dtype=np.int64)
            offs = []
            for l, l1, l2 in cgu.SparseLtuples.get_iter(L, llls):
                offs.append(t_ff[l])
                t_ff[l] += taus[l1] * taus[l2]
            out[f"{mode}_{L}_{tag}_taus"] = np.asarray(taus, dtype=np.int64)
            out[f"{mode}_{L}_{tag}_tFF"] = t_ff
            out[f"{mode}_{L}_{tag}_toffsets"] = np.asarray(offs, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "index_layer.npz"), **out)
    return len(out)


def cg_fixtures(cgu):
    import ClebschGordan
    out = {}
    L = 4
    D = ClebschGordan.precompute(L)
    for idx, mat in D.items():
        l = idx % (L + 1)
        l2 = (idx // (L + 1)) % (L + 1)
        l1 = idx // (L + 1) ** 2
        out[f"dense_L4_{l1}_{l2}_{l}"] = np.asarray(mat, dtype=np.float64)
    # band tables exactly as the reference's CPU builder lays them out (CGutils.py:161-177)
    for L in (3, 6):
        llls, _ = cgu.SparseLtuples.sparse_rep_ltuples_sorted(cgu.SparseLtuples.compute_default_ltuples(L))
        out[f"band_default_{L}"] = cgu.SparseLtuples.precompute_CG_from_llls(L, llls).numpy()
    # moments of the big tables: cheap to store, sensitive to any wrong entry or sign
    for L in (10, 20):
        D = ClebschGordan.precompute(L)
        keys = sorted(D.keys())
        out[f"dense_L{L}_keys"] = np.asarray(keys, dtype=np.int64)
        out[f"dense_L{L}_sum"] = np.asarray([D[k].sum() for k in keys])
        out[f"dense_L{L}_abs"] = np.asarray([np.abs(D[k]).sum() for k in keys])
        w = [np.cos(np.arange(D[k].size).reshape(D[k].shape) * 0.37) for k in keys]
        out[f"dense_L{L}_wsum"] = np.asarray([(D[k] * w[i]).sum() for i, k in enumerate(keys)])
    np.savez_compressed(os.path.join(HERE, "cg_coefficients.npz"), **out)
    return len(out)


def gen_fs(taus, B, seed):
    """Inputs of the reference's own test (CGNet/test.py:33-37): uniform [0,10) with numpy's seeded global RNG."""
    np.random.seed(seed)
    return [np.random.rand(B, taus[l], 2 * l + 1, 2) * 10 for l in range(len(taus))]


def gen_normal(taus, B, seed):
    rng = np.random.RandomState(seed)
    return [rng.randn(B, taus[l], 2 * l + 1, 2) for l in range(len(taus))]


def _grads(fs, B):
    """Flat gradient of the inputs; a fragment no pair uses gets zeros (autograd leaves its .grad unset)."""
    return torch.cat([(torch.zeros_like(f) if f.grad is None else f.grad).reshape(B, -1, 2) for f in fs], 1).numpy()


def layer_case(cgu, cgpy, name, taus, tau_out, B, mode, inputs, store_ff, cgdict_cache):
    L = len(taus) - 1
    if L not in cgdict_cache:
        cgdict_cache[L] = cgu.ClebschGordanDict(L)
    ltuples = {"default": None, "mst": "mst", "debug": "debug"}[mode]
    cg = cgpy.CG_sparse_py(L, taus, ltuples=ltuples, precomputed_CG=cgdict_cache[L])
    numcols = cg.t_FF
    bn = cgpy.MyBatchNormList(L, numcols, init="debug")            # seeds numpy with 0, stds ~ U[0,1)
    bn.eval()
    torch.manual_seed(0)                                             # CGBN_base.reset_parameters, init='debug'
    wlen = int(np.sum(np.asarray(numcols) * np.asarray(tau_out)))
    W = (0.05 * torch.rand(wlen, 2, dtype=torch.float)).requires_grad_(True)

    fs = [torch.tensor(a, dtype=torch.float, requires_grad=True) for a in inputs]
    rng = np.random.RandomState(1234)

    def mixing(new_fs):                                              # CGBN_base.forward, CG_layers_python.py:259-266
        outs, offset = [], 0
        for l, fl in enumerate(new_fs):
            wl = W[offset:(offset + numcols[l] * tau_out[l]), :].view(tau_out[l], numcols[l], 2)
            offset += numcols[l] * tau_out[l]
            outs.append(cgu.Complex_bmm(wl.repeat(B, 1, 1, 1), fl))
        return outs

    out = {}
    out["taus"] = np.asarray(taus, dtype=np.int64)
    out["tau_out"] = np.asarray(tau_out, dtype=np.int64)
    out["llls"] = np.asarray(cg.llls, dtype=np.int64)
    out["F"] = torch.cat([f.detach().reshape(B, -1, 2) for f in fs], 1).numpy()
    out["W"] = W.detach().numpy()
    stds_flat = torch.cat([p.detach().flatten() for p in bn.stds]).numpy()
    out["stds"] = stds_flat

    # (1) the CG product alone, with gradient of a fixed linear functional
    ff = cg(list(fs))
    ff_flat = torch.cat([f.reshape(B, -1, 2) for f in ff], 1)
    g_ff = torch.tensor(rng.randn(*ff_flat.shape), dtype=torch.float)
    (ff_flat * g_ff).sum().backward()
    if store_ff:
        out["FF"] = ff_flat.detach().numpy()
        out["gFF"] = g_ff.numpy()
    else:  # keep the fixture small: per-fragment Frobenius norms and a fixed random projection
        out["FF_fragnorm"] = np.asarray([float(f.detach().norm()) for f in ff])
        out["FF_proj"] = np.asarray(float((ff_flat.detach().double() * g_ff.double()).sum()))
        out["gFF_seed"] = np.asarray(1234)
    out["cg_gF"] = _grads(fs, B)
    for f in fs:
        f.grad = None

    # (2) product -> mixing, no normalisation
    o = mixing(cg(list(fs)))
    o_flat = torch.cat([f.reshape(B, -1, 2) for f in o], 1)
    g_o = torch.tensor(rng.randn(*o_flat.shape), dtype=torch.float)
    (o_flat * g_o).sum().backward()
    out["nobn_O"] = o_flat.detach().numpy()
    out["gO"] = g_o.numpy()
    out["nobn_gF"] = _grads(fs, B)
    out["nobn_gW"] = W.grad.numpy().copy()
    W.grad = None
    for f in fs:
        f.grad = None

    # (3) product -> fragment norm (eval: stored stds) -> mixing
    o = mixing(bn(cg(list(fs))))
    o_flat = torch.cat([f.reshape(B, -1, 2) for f in o], 1)
    (o_flat * g_o).sum().backward()
    out["bneval_O"] = o_flat.detach().numpy()
    out["bneval_gF"] = _grads(fs, B)
    out["bneval_gW"] = W.grad.numpy().copy()
    W.grad = None
    for f in fs:
        f.grad = None

    # (4) training step of the norm: transcription of MyBatchNormList.forward lines 172-183 without `.cuda()`
    cnt = 1.0
    new_fs = cg(list(fs))
    new_stds = []
    normed = []
    for l in range(L + 1):
        fl = new_fs[l]
        npv = fl.detach().numpy().copy()
        norm = np.linalg.norm(npv, ord=2, axis=3)
        std = torch.tensor(np.std(norm, axis=(0, 2)))
        s = bn.stds[l].detach().clone()
        s *= cnt / (cnt + 1.)
        s[:, 0, 0] += std / (cnt + 1)
        new_stds.append(s)
        normed.append(fl / torch.max(bn.eps, s))
    o = mixing(normed)
    o_flat = torch.cat([f.reshape(B, -1, 2) for f in o], 1)
    (o_flat * g_o).sum().backward()
    out["harness_bntrain_stds"] = torch.cat([s.flatten() for s in new_stds]).numpy()
    out["harness_bntrain_O"] = o_flat.detach().numpy()
    out["harness_bntrain_gF"] = _grads(fs, B)
    out["harness_bntrain_gW"] = W.grad.numpy().copy()
    return {f"{name}/{k}": v for k, v in out.items()}


def layer_fixtures(cgu, cgpy):
    cache = {}
    out = {}
    cases = [
        # name, taus, tau_out, B, pair mode, inputs, store FF
        ("t21_mst", [2, 1], [2, 1], 2, "mst", gen_fs([2, 1], 2, 0), True),           # CGNet/test.py:130
        ("t21_default", [2, 1], [2, 1], 2, "default", gen_fs([2, 1], 2, 0), True),
        ("t32111_default", [3, 2, 1, 1, 1], [3, 2, 1, 1, 1], 1, "default", gen_fs([3, 2, 1, 1, 1], 1, 0), True),  # :81
        ("t32111_mst", [3, 2, 1, 1, 1], [2, 2, 2, 1, 1], 2, "mst", gen_fs([3, 2, 1, 1, 1], 2, 1), True),
        ("t211_default", [2, 1, 1], [2, 1, 1], 2, "default", gen_normal([2, 1, 1], 2, 5), True),
        ("t2222_debug", [2, 2, 2, 2], [3, 1, 2, 2], 3, "debug", gen_normal([2, 2, 2, 2], 3, 6), True),
        ("L5t4_default", [4] * 6, [4] * 6, 3, "default", gen_normal([4] * 6, 3, 7), False),
        ("L6ragged_mst", [3, 1, 4, 1, 5, 2, 2], [2, 3, 1, 4, 1, 2, 3], 2, "mst", gen_normal([3, 1, 4, 1, 5, 2, 2], 2, 8), False),
    ]
    for name, taus, tau_out, B, mode, inputs, store_ff in cases:
        out.update(layer_case(cgu, cgpy, name, taus, tau_out, B, mode, inputs, store_ff, cache))
    np.savez_compressed(os.path.join(HERE, "layer_cases.npz"), **out)
    return len(out)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref", default=os.environ.get("CGNET_REFERENCE"), required=os.environ.get("CGNET_REFERENCE") is None,
                    help="path of a zlin7/CGNet checkout (or set CGNET_REFERENCE)")
    args = ap.parse_args()
    cgu, cgpy = import_reference(args.ref)
    n1 = index_fixtures(cgu)
    n2 = cg_fixtures(cgu)
    n3 = layer_fixtures(cgu, cgpy)
    print(f"wrote index_layer.npz ({n1} arrays), cg_coefficients.npz ({n2}), layer_cases.npz ({n3})")
    print("versions:", "numpy", np.__version__, "torch", torch.__version__, "scipy", __import__("scipy").__version__)
