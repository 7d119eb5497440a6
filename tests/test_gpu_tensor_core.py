"""The tensor-core (tcgen05 + tensor memory + bulk async copy, 3xTF32) variant of the fused forward against the CPU
oracle and against the CUDA-core variant.  Tolerance as everywhere: relative Frobenius error per fragment < 1e-4."""
import ctypes
import os

import numpy as np
import pytest
import torch

from helpers import assert_fragments_close, assert_weights_close, make_case, oracle_layer

pytestmark = pytest.mark.gpu

CASES = [
    # taus, tau_out, B, pair mode
    ([8] * 4, [8] * 4, 40, "default"),
    ([4] * 3, [16] * 3, 5, "default"),
    ([16] * 6, [16] * 6, 33, "default"),
    ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default"),      # ragged channel counts, partial tiles, N' padded to 16 / 32
    ([8] * 8, [12] * 8, 64, "mst"),
    ([2] * 5, [8] * 5, 3, "default"),                   # tile edge 2
    ([8] * 11, [32] * 11, 20, "default"),
]


def _forward(plan, case, bn, training, tc):
    from cgnet_b200 import _lib
    dev = torch.device("cuda", 0)
    os.environ["CGB200_TC"] = "1" if tc else "0"
    try:
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if training else 0)
        O = plan.layer_fwd(F, W, stds, 2.0, 1e-5, flags)
        torch.cuda.synchronize()
        st = ctypes.c_int32(-1)
        _lib.check(_lib.load().cgb200_plan_status(plan.handle, st), "cgb200_plan_status")
        assert st.value == 0, "a bounded wait inside the tensor-core kernel ran out"
        return O.cpu().numpy(), None if stds is None else stds.cpu().numpy()
    finally:
        os.environ.pop("CGB200_TC", None)


@pytest.mark.parametrize("bn,training", [(False, False), (True, True)])
@pytest.mark.parametrize("taus,tau_out,B,mode", CASES)
def test_tensor_core_forward(taus, tau_out, B, mode, bn, training):
    from cgnet_b200 import get_plan
    case = make_case(taus, tau_out, B, mode, seed=51)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    if plan.tile not in (2, 4):
        pytest.skip(f"tile edge {plan.tile}: the tensor-core forward is built for 2 and 4")
    O_want, _, _, stds_want = oracle_layer(case, bn, training, cnt=2.0)
    O_tc, stds_tc = _forward(plan, case, bn, training, tc=True)
    assert_fragments_close(O_tc, O_want, tau_out, "O (tensor-core forward) vs oracle")
    O_cc, _ = _forward(plan, case, bn, training, tc=False)
    assert_fragments_close(O_tc, O_cc, tau_out, "O (tensor-core forward) vs CUDA-core forward")
    if training:
        np.testing.assert_allclose(stds_tc, stds_want, rtol=2e-5, atol=1e-7)


def test_tensor_core_forward_is_deterministic():
    from cgnet_b200 import get_plan
    case = make_case([8] * 5, [8] * 5, 50, "default", seed=52)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], torch.device("cuda", 0))
    a, _ = _forward(plan, case, True, False, tc=True)
    b, _ = _forward(plan, case, True, False, tc=True)
    assert np.array_equal(a, b)


def _weight_gradient(plan, case, bn, tc):
    from cgnet_b200 import _lib
    dev = torch.device("cuda", 0)
    os.environ["CGB200_TC_GW"] = "1" if tc else "0"
    try:
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        _, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT if bn else 0, gO)
        torch.cuda.synchronize()
        st = ctypes.c_int32(-1)
        _lib.check(_lib.load().cgb200_plan_status(plan.handle, st), "cgb200_plan_status")
        assert st.value == 0, "a bounded wait inside the tensor-core kernel ran out"
        return gW.cpu().numpy()
    finally:
        os.environ.pop("CGB200_TC_GW", None)


GW_CASES = CASES + [
    ([5] * 6, [5] * 6, 40, "default"),            # tile edge 5: two cells per block, generator warps split the rows 3 + 2
    ([5] * 11, [5] * 11, 100, "default"),         # the benchmark layer: sample groups sliced over blocks, partial sums reduced
    ([10] * 4, [7] * 4, 33, "default"),
    ([5, 3, 10, 5, 1], [4, 5, 2, 7, 5], 70, "mst"),
]


@pytest.mark.parametrize("bn", [False, True])
@pytest.mark.parametrize("taus,tau_out,B,mode", GW_CASES)
def test_tensor_core_weight_gradient(taus, tau_out, B, mode, bn):
    """gW from the tcgen05 weight-gradient kernel (3xTF32, contraction over samples and m in tensor memory) against the
    oracle's autograd gradient and against the CUDA-core kernel."""
    from cgnet_b200 import get_plan
    import cg_oracle as o
    case = make_case(taus, tau_out, B, mode, seed=53)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    if plan.tile not in (4, 5):
        pytest.skip(f"tile edge {plan.tile}: the tensor-core weight gradient is built for 4 and 5")
    t_ff, _ = o.tau_ff_and_offsets(case["lmax"], taus, case["llls"])
    _, _, gW_want, _ = oracle_layer(case, bn, False, cnt=2.0)
    gW_tc = _weight_gradient(plan, case, bn, tc=True)
    assert_weights_close(gW_tc, gW_want, t_ff, tau_out, "gW (tensor-core) vs oracle")
    gW_cc = _weight_gradient(plan, case, bn, tc=False)
    assert_weights_close(gW_tc, gW_cc, t_ff, tau_out, "gW (tensor-core) vs CUDA-core kernel")


def test_tensor_core_weight_gradient_is_deterministic():
    from cgnet_b200 import get_plan
    case = make_case([8] * 5, [16] * 5, 70, "default", seed=54)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], torch.device("cuda", 0))
    a = _weight_gradient(plan, case, True, tc=True)
    b = _weight_gradient(plan, case, True, tc=True)
    assert np.array_equal(a, b)


def _input_gradient(plan, case, bn, tc):
    from cgnet_b200 import _lib
    dev = torch.device("cuda", 0)
    os.environ["CGB200_TC_GF"] = "1" if tc else "0"
    try:
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        gF, _ = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT if bn else 0, gO)
        torch.cuda.synchronize()
        st = ctypes.c_int32(-1)
        _lib.check(_lib.load().cgb200_plan_status(plan.handle, st), "cgb200_plan_status")
        assert st.value == 0, "a bounded wait inside the tensor-core kernel ran out"
        return gF.cpu().numpy()
    finally:
        os.environ.pop("CGB200_TC_GF", None)


@pytest.mark.parametrize("bn", [False, True])
@pytest.mark.parametrize("taus,tau_out,B,mode", CASES + [([4] * 15, [20] * 15, 33, "mst"), ([8] * 4, [40] * 4, 9, "default")])
def test_tensor_core_input_gradient(taus, tau_out, B, mode, bn):
    """gF from the input-gradient kernel whose gFF tiles come from tcgen05 MMAs (3xTF32, accumulator in tensor memory,
    moved to shared memory for the CG contraction) against the oracle's autograd gradient and the CUDA-core kernel."""
    from cgnet_b200 import get_plan
    case = make_case(taus, tau_out, B, mode, seed=55)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    if plan.tile != 4:
        pytest.skip(f"tile edge {plan.tile}: the tensor-core input gradient is built for 4")
    _, gF_want, _, _ = oracle_layer(case, bn, False, cnt=2.0)
    gF_tc = _input_gradient(plan, case, bn, tc=True)
    assert_fragments_close(gF_tc, gF_want, taus, "gF (tensor-core phase 1) vs oracle")
    gF_cc = _input_gradient(plan, case, bn, tc=False)
    assert_fragments_close(gF_tc, gF_cc, taus, "gF (tensor-core phase 1) vs CUDA-core kernel")


def test_tensor_core_input_gradient_is_deterministic():
    from cgnet_b200 import get_plan
    case = make_case([8] * 5, [16] * 5, 70, "default", seed=56)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], torch.device("cuda", 0))
    a = _input_gradient(plan, case, True, tc=True)
    b = _input_gradient(plan, case, True, tc=True)
    assert np.array_equal(a, b)
