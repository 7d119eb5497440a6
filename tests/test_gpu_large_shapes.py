"""Parity at the layer shapes of the larger benchmark workloads, where the tensor-core kernels run and where the error of
their 3xTF32 products (fp32 accumulation inside the tensor core) is largest because the contraction is longest:

    lmax 14, 16 channels (6 input channels for the first layer)   the six-layer training network
    lmax 20, 32 channels, MST pair lists, full channel product       the reference's 'mst' mode (CG_layers.py:226-230)
    lmax 20, 32 channels, MST pair lists, channel-wise product      the depthwise extension (no reference counterpart)
    lmax 10, 64 channels                                             contraction length up to 180 k complex channels
    lmax 1, 1200 channels in degree 0                                contraction length 1.44 M: beyond the largest sweep point

Every call goes through the C ABI; the checker is the fp64 CPU oracle at a small batch.  Tolerance: relative Frobenius
error per fragment < 1e-4 (helpers.TOL); the measured errors are printed (pytest -s) so that the margin is on record.
"""
import functools

import numpy as np
import pytest
import torch

import cg_oracle as o
from helpers import TOL, make_case, oracle_layer, rel_fro

pytestmark = pytest.mark.gpu

SHAPES = {
    "lmax14_first": ([6] * 15, [16] * 15, 2, "default", False),
    "lmax14_tau16": ([16] * 15, [16] * 15, 2, "default", False),
    "lmax20_tau32_mst": ([32] * 21, [32] * 21, 1, "mst", False),
    "lmax20_tau32_mst_depthwise": ([32] * 21, [32] * 21, 3, "mst", True),
    "lmax10_tau64": ([64] * 11, [64] * 11, 1, "default", False),
    "long_contraction": ([1200, 4], [16, 16], 2, "default", False),
}


@functools.lru_cache(maxsize=None)
def case_and_oracle(name, training):
    taus, tau_out, B, mode, dw = SHAPES[name]
    case = make_case(taus, tau_out, B, mode, seed=71, depthwise=dw)
    case.pop("gFF")   # only the two-pass tests need a cotangent of the product; it is the largest array by far
    return case, oracle_layer(case, True, training, cnt=3.0)


def worst(got, want, taus):
    """Largest per-fragment relative Frobenius error of a flat (B, N, 2) activation."""
    off, w = 0, 0.0
    for l, t in enumerate(taus):
        n = int(t) * (2 * l + 1)
        if n:
            w = max(w, rel_fro(got[:, off:off + n], want[:, off:off + n]))
        off += n
    return w


def worst_w(got, want, t_ff, tau_out):
    off, w = 0, 0.0
    for l in range(len(t_ff)):
        n = int(t_ff[l]) * int(tau_out[l])
        if n:
            w = max(w, rel_fro(got[off:off + n], want[off:off + n]))
        off += n
    return w


@pytest.mark.parametrize("training", [False, True])
@pytest.mark.parametrize("name", sorted(SHAPES))
def test_fused_layer_at_benchmark_shapes(name, training, capsys):
    from cgnet_b200 import _lib, get_plan
    dev = torch.device("cuda", 0)
    case, (O_want, gF_want, gW_want, stds_want) = case_and_oracle(name, training)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev, depthwise=case["depthwise"])
    assert plan.t_ff() == [int(x) for x in case["t_ff"]]
    F = torch.tensor(case["F"], device=dev)
    W = torch.tensor(case["W"], device=dev)
    gO = torch.tensor(case["gO"], device=dev)
    stds = torch.tensor(case["stds"], device=dev)
    flags = _lib.FN_PRESENT | (_lib.FN_UPDATE if training else 0)
    O = plan.layer_fwd(F, W, stds, 3.0, 1e-5, flags)
    gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
    plan.check_status()
    errs = {"O": worst(O.cpu().numpy(), O_want, case["tau_out"]), "gF": worst(gF.cpu().numpy(), gF_want, case["taus"]),
            "gW": worst_w(gW.cpu().numpy(), gW_want, case["t_ff"], case["tau_out"])}
    if training:
        errs["stds"] = rel_fro(stds.cpu().numpy(), stds_want)
    with capsys.disabled():
        kmax = int(max(case["t_ff"]))
        print(f"\n[parity] {name} ({'training' if training else 'stored'} norm, tile {plan.tile}, longest contraction "
              f"{kmax} complex channels): " + ", ".join(f"{k} {v:.2e}" for k, v in errs.items()))
    for k, v in errs.items():
        assert v < TOL, f"{name}: {k} relative Frobenius error {v:.3e} >= {TOL}"


def test_tensor_core_variants_at_long_contractions():
    """The kernels that are on by default at these widths are the tensor-core ones; hold each of them, by option, to the
    CUDA-core variant of the same plan on the lmax-10, 64-channel shape (K up to 180 k complex channels)."""
    from cgnet_b200 import _lib, get_plan
    dev = torch.device("cuda", 0)
    case, (O_want, gF_want, gW_want, _) = case_and_oracle("lmax10_tau64", False)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev)
    assert plan.tile == 4
    F = torch.tensor(case["F"], device=dev)
    W = torch.tensor(case["W"], device=dev)
    gO = torch.tensor(case["gO"], device=dev)
    stds = torch.tensor(case["stds"], device=dev)
    out = {}
    for tc in (0, 1):
        for opt in (_lib.OPT_TC_FWD, _lib.OPT_TC_GRAD_W, _lib.OPT_TC_GRAD_F):
            plan.set_option(opt, tc)
        try:
            O = plan.layer_fwd(F, W, stds, 3.0, 1e-5, _lib.FN_PRESENT)
            gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
            plan.check_status()
        finally:
            for opt in (_lib.OPT_TC_FWD, _lib.OPT_TC_GRAD_W, _lib.OPT_TC_GRAD_F):
                plan.set_option(opt, _lib.AUTO)
        out[tc] = (O.cpu().numpy(), gF.cpu().numpy(), gW.cpu().numpy())
    for tc in (0, 1):
        O, gF, gW = out[tc]
        tag = "tensor-core" if tc else "CUDA-core"
        assert worst(O, O_want, case["tau_out"]) < TOL, tag
        assert worst(gF, gF_want, case["taus"]) < TOL, tag
        assert worst_w(gW, gW_want, case["t_ff"], case["tau_out"]) < TOL, tag


def test_tensor_core_weight_gradient_over_a_long_batch():
    """The weight gradient contracts over (sample, m): with a large batch in one slice the tensor-core kernel sums
    thousands of accumulation steps per output.  Held to the CUDA-core kernel of the same plan, which sums in
    registers with rounded adds (no oracle needed: the product for 2048 samples would not fit the CPU checker)."""
    from cgnet_b200 import _lib, get_plan
    dev = torch.device("cuda", 0)
    taus, tau_out, B = [16] * 5, [16] * 5, 2048
    small = make_case(taus, tau_out, 2, "default", seed=72)
    plan = get_plan(small["lmax"], taus, tau_out, small["llls"], dev)
    assert plan.tile == 4
    rng = np.random.RandomState(73)
    F = torch.tensor(rng.randn(B, plan.n_F, 2).astype(np.float32), device=dev)
    gO = torch.tensor(rng.randn(B, plan.n_O, 2).astype(np.float32), device=dev)
    W = torch.tensor(small["W"], device=dev)
    stds = torch.tensor(small["stds"], device=dev)
    got = {}
    for tc in (0, 1):
        plan.set_option(_lib.OPT_TC_GRAD_W, tc)
        try:
            _, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO, need_gF=False)
            plan.check_status()
        finally:
            plan.set_option(_lib.OPT_TC_GRAD_W, _lib.AUTO)
        got[tc] = gW.cpu().numpy()
    err = worst_w(got[1], got[0], small["t_ff"], tau_out)
    print(f"\n[parity] weight gradient over {B} samples, tensor cores vs CUDA cores: {err:.2e}")
    assert err < TOL
