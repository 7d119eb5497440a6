"""Lane sharing in a short last sample group (CGB200_OPT_SHORT_GROUP): a batch whose last group of 32 holds at most 16
samples lets the idle lanes of that group take rows of the work instead of repeating it for empty sample slots.  The
input gradient keeps every element's order of operations, so its bits must not change; the weight gradient sums the
lanes in another order and is held to the parity tolerance.  Shapes cover the tile edges 5 (benchmark layer), 4 with the
mid-gradient GEMM, 4 without it, 3, 1 and the depthwise product."""
import numpy as np
import pytest
import torch

from helpers import assert_fragments_close, assert_weights_close, make_case, oracle_layer

pytestmark = pytest.mark.gpu

SHAPES = [   # (taus, tau_out, mode, depthwise, options held fixed for both runs)
    ([5] * 5, [5] * 5, "default", False, {}),
    ([16] * 4, [16] * 4, "default", False, {}),                 # mid-gradient GEMM + gather
    ([16] * 4, [16] * 4, "default", False, {"OPT_GRAD_MID_GEMM": 0}),
    ([8, 7, 0, 6], [6, 0, 8, 4], "default", False, {}),
    ([3] * 4, [3] * 4, "mst", False, {}),
    ([1, 1, 1], [1, 1, 1], "default", False, {}),
    ([8] * 5, [8] * 5, "mst", True, {}),
]


def _backward(plan, case, options):
    from cgnet_b200 import _lib
    dev = plan.device
    for opt, v in options.items():
        plan.set_option(getattr(_lib, opt), v)
    try:
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev)
        gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
        plan.check_status()
        return gF.cpu().numpy(), gW.cpu().numpy()
    finally:
        for opt in options:
            plan.set_option(getattr(_lib, opt), _lib.AUTO)


@pytest.mark.parametrize("B", [1, 4, 7, 36, 40, 48, 100])
@pytest.mark.parametrize("shape", range(len(SHAPES)))
def test_input_gradient_bits_do_not_depend_on_lane_sharing(shape, B):
    from cgnet_b200 import get_plan
    taus, tau_out, mode, depthwise, fixed = SHAPES[shape]
    case = make_case(taus, tau_out, B, mode, seed=31 + shape, depthwise=depthwise)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0), depthwise=depthwise)
    shared = _backward(plan, case, dict(fixed))
    plain = _backward(plan, case, dict(fixed, OPT_SHORT_GROUP=0))
    assert np.array_equal(shared[0].view(np.uint32), plain[0].view(np.uint32)), "gF bits changed with lane sharing"
    assert_weights_close(shared[1], plain[1], case["t_ff"], tau_out, "gW, lane sharing on/off")
    if B <= 40:
        _, gF_want, gW_want, _ = oracle_layer(case, True, False)
        assert_fragments_close(shared[0], gF_want, taus, "gF vs oracle")
        assert_weights_close(shared[1], gW_want, case["t_ff"], tau_out, "gW vs oracle")
