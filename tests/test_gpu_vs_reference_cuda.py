"""Our kernels against the reference project's own CUDA kernels on the same GPU and the same seeded inputs.

The reference extension `CG_cuda_ops` (CGNet/cudaCG, unmodified sources) is compiled for sm_100a by
`python oracle/build_ref_cuda.py` into oracle/_ref/cuda_build/ (git-ignored, shipped with the tree).  Its six functions
are called directly with index tensors laid out as CGNet/CG_layers.py builds them (:244-250, :104-108); the reference's
Python files are not needed.  Skipped when the extension has not been built.  Tolerance: relative Frobenius error per
fragment < 1e-4 (fp32 on both sides)."""
import numpy as np
import pytest
import torch

import ref_cuda_driver as refdrv
from helpers import assert_fragments_close, assert_weights_close, make_case

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def ref_ops():
    if not refdrv.available():
        pytest.skip("reference CUDA extension not built (python oracle/build_ref_cuda.py)")
    return refdrv.load_ops()


def dev():
    return torch.device("cuda", 0)


def RefLayer(ops, case):
    """The reference's index tensors and kernel calls for one layer case (oracle/ref_cuda_driver.py)."""
    return refdrv.RefLayer.from_case(ops, case, dev())


CASES = [
    ([2, 1], [2, 1], 2, "mst"),
    ([3, 2, 1, 1, 1], [3, 2, 1, 1, 1], 1, "default"),
    ([4] * 6, [4] * 6, 3, "default"),
    ([3, 1, 4, 1, 5, 2, 2], [2, 3, 1, 4, 1, 2, 3], 2, "mst"),
    ([8] * 6, [8] * 6, 32, "default"),          # single layer lmax 5, 8 channels, batch 32
    ([5] * 11, [5] * 11, 100, "default"),       # one layer of the 5-layer lmax-10 classifier at its batch of 100
    ([1] * 11, [5] * 11, 100, "default"),       # its first layer
    ([4] * 11, [3] * 11, 5, "mst"),
    ([6] * 15, [16] * 15, 4, "default"),        # first layer of the lmax-14 training network (6 input channels)
    ([16] * 15, [16] * 15, 3, "default"),       # its other layers: tensor-core forward and weight gradient
    ([32] * 21, [32] * 21, 2, "mst"),           # lmax 20, 32 channels, MST pairs with the full channel product
    ([64] * 11, [64] * 11, 2, "default"),       # lmax 10, 64 channels
]


@pytest.mark.parametrize("taus,tau_out,B,mode", CASES)
def test_cg_table_and_product_match_reference_kernels(ref_ops, taus, tau_out, B, mode):
    from cgnet_b200 import get_plan
    case = make_case(taus, tau_out, B, mode, seed=41)
    ref = RefLayer(ref_ops, case)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev())
    from cgnet_b200.cg_layers import _precomputeCG_cuda
    ours_cg, _ = _precomputeCG_cuda(case["lmax"], case["llls"], dev())
    torch.cuda.synchronize()
    np.testing.assert_allclose(ours_cg.cpu().numpy(), ref.CG.cpu().numpy(), atol=3e-7, rtol=0)
    F = torch.tensor(case["F"], device=dev())
    gFF = torch.tensor(case["gFF"], device=dev())
    assert_fragments_close(plan.cg_product_fwd(F).cpu().numpy(), ref.product_fwd(F).cpu().numpy(), ref.t_ff, "FF vs reference kernel")
    assert_fragments_close(plan.cg_product_bwd(F, gFF).cpu().numpy(), ref.product_bwd(F, gFF).cpu().numpy(), taus,
                           "product gF vs reference kernel")


@pytest.mark.parametrize("bn,training", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("taus,tau_out,B,mode", CASES)
def test_layer_matches_reference_kernels(ref_ops, taus, tau_out, B, mode, bn, training):
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, mode, seed=42)
    ref = RefLayer(ref_ops, case)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev())
    F = torch.tensor(case["F"], device=dev())
    W = torch.tensor(case["W"], device=dev())
    gO = torch.tensor(case["gO"], device=dev())
    flags = (1 if bn else 0) | (2 if training else 0)
    cnt, eps = 2.0, 1e-5

    r_stds = torch.tensor(case["stds"], device=dev()) if bn else None
    r_FF = ref.product_fwd(F)
    r_O = ref.mix_fwd(r_FF, W, r_stds, cnt, eps, flags)
    r_gFF, r_gW = ref.mix_bwd(gO, r_FF, W, r_stds, cnt, eps, flags)
    r_gF = ref.product_bwd(F, r_gFF)
    torch.cuda.synchronize()

    for fused in (False, True):
        stds = torch.tensor(case["stds"], device=dev()) if bn else None
        if fused:
            O = plan.layer_fwd(F, W, stds, cnt, eps, flags)
            gF, gW = plan.layer_bwd(F, W, stds, eps, flags & _lib.FN_PRESENT, gO)
        else:
            FF = plan.cg_product_fwd(F)
            O = plan.fn_wmm_fwd(FF, W, stds, cnt, eps, flags)
            gFF, gW = plan.fn_wmm_bwd(gO, FF, W, stds, eps, flags & _lib.FN_PRESENT)
            gF = plan.cg_product_bwd(F, gFF)
        tag = "fused" if fused else "two-pass"
        assert_fragments_close(O.cpu().numpy(), r_O.cpu().numpy(), tau_out, f"O ({tag}) vs reference kernels")
        assert_weights_close(gW.cpu().numpy(), r_gW.cpu().numpy(), ref.t_ff, tau_out, f"gW ({tag}) vs reference kernels")
        assert_fragments_close(gF.cpu().numpy(), r_gF.cpu().numpy(), taus, f"gF ({tag}) vs reference kernels")
        if training:
            np.testing.assert_allclose(stds.cpu().numpy(), r_stds.cpu().numpy(), rtol=2e-5, atol=1e-7)


def _time_ms(fn, reps=10, warm=3):
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(reps):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / reps


SPEED_CASES = [
    ("benchmark layer (lmax 10, tau 5 -> 5, batch 100)", [5] * 11, [5] * 11, 100),
    ("benchmark first layer (lmax 10, tau 1 -> 5, batch 100)", [1] * 11, [5] * 11, 100),
    ("single layer lmax 5, tau 8, batch 32", [8] * 6, [8] * 6, 32),
]


@pytest.mark.parametrize("name,taus,tau_out,B", SPEED_CASES)
def test_layer_is_faster_than_reference_kernels(ref_ops, name, taus, tau_out, B, capsys):
    """Forward + backward of one layer with training-mode norm: the fused path and the reference's four kernel calls
    (product, norm + mixing, their two backward calls, with the zero-filled outputs the reference's modules allocate on
    every call, CGNet/CG_layers.py:262-286,126-160), timed with CUDA events on the same GPU.  The results of the two paths
    are compared by the parity tests above; this one records the ratio and fails if the fused path is not faster."""
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, "default", seed=43)
    ref = RefLayer(ref_ops, case)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev())
    F = torch.tensor(case["F"], device=dev())
    W = torch.tensor(case["W"], device=dev())
    gO = torch.tensor(case["gO"], device=dev())
    cnt, eps, flags = 2.0, 1e-5, 3
    r_stds = torch.tensor(case["stds"], device=dev())
    o_stds = r_stds.clone()

    def run_ref():
        FF = ref.product_fwd(F)
        ref.mix_fwd(FF, W, r_stds, cnt, eps, flags)
        gFF, _ = ref.mix_bwd(gO, FF, W, r_stds, cnt, eps, flags)
        ref.product_bwd(F, gFF)

    def run_ours():
        plan.layer_fwd(F, W, o_stds, cnt, eps, flags)
        plan.layer_bwd(F, W, o_stds, eps, flags & _lib.FN_PRESENT, gO)

    t_ref, t_ours = _time_ms(run_ref), _time_ms(run_ours)
    with capsys.disabled():
        print(f"\n[speed] {name}: reference kernels {t_ref:.3f} ms, fused path {t_ours:.3f} ms, ratio {t_ref / t_ours:.1f}x")
    assert t_ours < t_ref, f"{name}: fused path {t_ours:.3f} ms is not faster than the reference kernels {t_ref:.3f} ms"
