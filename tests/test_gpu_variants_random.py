"""Seeded random layer shapes (ragged channel counts, empty fragments, odd batch sizes, both pair modes, free and
forced tile edge): the fused layer with every kernel variant at its default against the same layer with the
memory-for-recomputation variants switched off (kept tiles, mid-gradient GEMM, split contraction, lane sharing of a
short last group) and, for the smaller cases, against the fp64 oracle.  The variants change the order of some sums,
so the comparison is the per-fragment tolerance of the parity tests, not bit equality."""
import numpy as np
import pytest
import torch

from helpers import assert_fragments_close, assert_weights_close, make_case, oracle_layer

pytestmark = pytest.mark.gpu


def _random_case(seed):
    rng = np.random.RandomState(1000 + seed)
    lmax = int(rng.randint(1, 7))
    wide = bool(rng.randint(0, 2))
    hi_in, hi_out = (21, 25) if wide else (9, 9)
    taus = [int(rng.randint(0, hi_in)) for _ in range(lmax + 1)]
    tau_out = [int(rng.randint(0, hi_out)) for _ in range(lmax + 1)]
    taus[int(rng.randint(0, lmax + 1))] = max(taus[0], 3)        # at least one populated fragment on each side
    tau_out[int(rng.randint(0, lmax + 1))] = max(tau_out[0], 4)
    B = int(rng.choice([1, 3, 4, 17, 32, 33, 36, 40, 65, 70]))
    mode = "mst" if rng.randint(0, 3) == 0 else "default"
    tile = int(rng.choice([0, 0, 4]))
    return taus, tau_out, B, mode, tile


def _run(plan, case, options):
    from cgnet_b200 import _lib
    dev = plan.device
    for opt, v in options.items():
        plan.set_option(opt, v)
    try:
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev)
        if not options and plan.keeps_mid(F.shape[0]):   # defaults: also hand the forward's workspace to the backward
            O, ws = plan.layer_fwd(F, W, stds, 2.0, 1e-5, _lib.FN_PRESENT | _lib.FN_UPDATE, keep=True)
            gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO, kept=ws)
        else:
            O = plan.layer_fwd(F, W, stds, 2.0, 1e-5, _lib.FN_PRESENT | _lib.FN_UPDATE)
            gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
        plan.check_status()
        return O.cpu().numpy(), stds.cpu().numpy(), gF.cpu().numpy(), gW.cpu().numpy()
    finally:
        for opt in options:
            plan.set_option(opt, _lib.AUTO)


@pytest.mark.parametrize("seed", range(40))
def test_default_variants_against_plain_variants(seed):
    from cgnet_b200 import _lib, get_plan
    import cg_oracle as o
    taus, tau_out, B, mode, tile = _random_case(seed)
    case = make_case(taus, tau_out, B, mode, seed=seed)
    try:
        plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0), tile=tile)
    except RuntimeError as e:   # a shape the library refuses (no triple produces an output, ...) is not this test's subject
        pytest.skip(str(e))
    t_ff, _ = o.tau_ff_and_offsets(case["lmax"], taus, case["llls"])
    assert plan.t_ff() == [int(t) for t in t_ff]
    new = _run(plan, case, {})
    plain = _run(plan, case, {_lib.OPT_FWD_KEEP_MID: 0, _lib.OPT_GRAD_MID_GEMM: 0, _lib.OPT_TC_FWD_SPLIT: 0, _lib.OPT_SHORT_GROUP: 0})
    tag = f"seed {seed}: taus {taus} -> {tau_out}, batch {B}, {mode}, tile {plan.tile}"
    assert_fragments_close(new[0], plain[0], tau_out, "O, " + tag)
    np.testing.assert_allclose(new[1], plain[1], rtol=2e-5, atol=1e-7, err_msg="stds, " + tag)
    assert_fragments_close(new[2], plain[2], taus, "gF, " + tag)
    assert_weights_close(new[3], plain[3], t_ff, tau_out, "gW, " + tag)
    if sum(int(t) * int(u) for t, u in zip(t_ff, tau_out)) * B < 4_000_000:   # the oracle stays within seconds
        O_want, gF_want, gW_want, stds_want = oracle_layer(case, True, True, cnt=2.0)
        assert_fragments_close(new[0], O_want, tau_out, "O vs oracle, " + tag)
        assert_fragments_close(new[2], gF_want, taus, "gF vs oracle, " + tag)
        assert_weights_close(new[3], gW_want, t_ff, tau_out, "gW vs oracle, " + tag)
        np.testing.assert_allclose(new[1], stds_want, rtol=2e-5, atol=1e-7)
