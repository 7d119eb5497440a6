"""The allocation-free forward entry point, cgb200_layer_fwd_static, against cgb200_layer_fwd.

Some hosts of this library cannot allocate device memory when they call it (a plugin inside another runtime's callback,
a process whose memory belongs to a foreign arena, a service that forbids cudaMalloc after start-up).  For them the
library carries its own fixed scratch array.  This test drives that entry point through the C ABI twice in a row - the
second call finds the array dirty from the first - and requires the same output as the ordinary entry point, which
gets a fresh workspace from the caller; it also checks that an over-sized request is refused with a message.

The file sorts last on purpose: should the fixed array ever misbehave, every other test has already run.
"""
import numpy as np
import pytest
import torch

from helpers import TOL, assert_fragments_close, make_case

pytestmark = pytest.mark.gpu


def _run_static(lib, plan, F, W, stds, cnt, flags, n_o):
    O = torch.empty(F.shape[0], n_o, 2, device=F.device, dtype=torch.float32)
    rc = lib.cgb200_layer_fwd_static(plan.handle, F.data_ptr(), W.data_ptr(), None if stds is None else stds.data_ptr(),
                                     cnt, 1e-5, flags, O.data_ptr(), F.shape[0], torch.cuda.current_stream().cuda_stream)
    return rc, O


def test_static_scratch_forward_matches_workspace_forward():
    from cgnet_b200 import _lib, get_plan
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    flags = _lib.FN_PRESENT | _lib.FN_UPDATE
    # two different shapes back to back, so the second call meets scratch left behind by a different layout
    for taus, tau_out, B, seed in (([5] * 6, [5] * 6, 37, 31), ([3, 1, 4, 2], [2, 3, 1, 4], 70, 32)):
        case = make_case(taus, tau_out, B, "default", seed=seed)
        plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev)
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        stds_ref = torch.tensor(case["stds"], device=dev)
        want = plan.layer_fwd(F, W, stds_ref, 1.0, 1e-5, flags)          # existing entry point, caller's workspace
        for call in range(2):
            stds = torch.tensor(case["stds"], device=dev)
            rc, got = _run_static(lib, plan, F, W, stds, 1.0, flags, plan.n_O)
            assert rc == 0, lib.cgb200_last_error()
            torch.cuda.synchronize()
            assert_fragments_close(got.cpu().numpy(), want.cpu().numpy(), tau_out, f"static forward, call {call}", tol=TOL)
            np.testing.assert_allclose(stds.cpu().numpy(), stds_ref.cpu().numpy(), rtol=1e-6, atol=0)


def test_static_scratch_rejects_oversized_requests():
    from cgnet_b200 import _lib, get_plan
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    case = make_case([8] * 8, [8] * 8, 4, "default", seed=33)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev)
    B = 8192   # far beyond what the built-in array can serve for this layer
    assert lib.cgb200_layer_fwd_workspace_bytes(plan.handle, B) > (8 << 20)
    F = torch.zeros(4, plan.n_F, 2, device=dev)   # never read: the call must refuse before launching anything
    W = torch.tensor(case["W"], device=dev)
    O = torch.zeros(4, plan.n_O, 2, device=dev)
    rc = lib.cgb200_layer_fwd_static(plan.handle, F.data_ptr(), W.data_ptr(), None, 1.0, 1e-5, 0, O.data_ptr(), B, None)
    assert rc == 4
    msg = lib.cgb200_last_error().decode()
    assert "scratch" in msg and str(8 << 20) in msg


def test_static_scratch_is_sized_by_the_forward_alone():
    """A batch whose forward scratch fits the built-in array although forward plus backward would not: the entry point
    must accept it (its limit is the forward's own need) and agree with the ordinary entry point."""
    from cgnet_b200 import _lib, get_plan
    lib = _lib.load()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B = 1600
    case = make_case([8] * 7, [8] * 7, 2, "default", seed=34)   # weights and statistics; the large batch is drawn below
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev)
    # the need of this forward (stored statistics: no tiles are kept) against the need of forward plus backward
    assert lib.cgb200_layer_fwd_workspace_bytes_for(plan.handle, B, _lib.FN_PRESENT) <= (8 << 20) < lib.cgb200_layer_workspace_bytes(plan.handle, B)
    F = torch.tensor(np.random.RandomState(35).randn(B, plan.n_F, 2).astype(np.float32), device=dev)
    W = torch.tensor(case["W"], device=dev)
    stds = torch.tensor(case["stds"], device=dev)
    want = plan.layer_fwd(F, W, stds, 1.0, 1e-5, _lib.FN_PRESENT)
    rc, got = _run_static(lib, plan, F, W, stds, 1.0, _lib.FN_PRESENT, plan.n_O)
    assert rc == 0, lib.cgb200_last_error()
    torch.cuda.synchronize()
    assert_fragments_close(got.cpu().numpy(), want.cpu().numpy(), case["tau_out"], "static forward, forward-sized scratch", tol=TOL)
