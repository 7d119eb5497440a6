"""The drop-in module `cgnet_b200.CG_cuda_ops` (the reference extension's six functions, same names and argument lists,
CGNet/cudaCG/cudaCG_all.cpp:207-215) driven exactly as the reference's Python layer drives its compiled extension:
caller-allocated zero-filled outputs and the seven int32 index tensors of CG_layers.py:244-250 / :104-108.  The same
driver object (oracle/ref_cuda_driver.py) is pointed once at this module and once at the reference's own extension
built from its unmodified sources, on identical tensors; results must agree to the parity tolerance (relative Frobenius
error per fragment < 1e-4), and with the library's own module path bit for bit (same kernels underneath)."""
import numpy as np
import pytest
import torch

import ref_cuda_driver as refdrv
from helpers import assert_fragments_close, assert_weights_close, make_case

pytestmark = pytest.mark.gpu

CASES = [
    ([2, 1], [2, 1], 2, "mst"),                       # the reference test's default invocation (CGNet/test.py:130)
    ([3, 2, 1, 1, 1], [3, 2, 1, 1, 1], 1, "default"),  # CGNet/test.py:81
    ([4] * 6, [4] * 6, 3, "default"),
    ([5] * 11, [5] * 11, 20, "default"),
    ([3, 1, 4, 1, 5, 2, 2], [2, 3, 1, 4, 1, 2, 3], 2, "mst"),
    ([6, 0, 3, 2], [2, 2, 0, 3], 4, "default"),        # empty fragments on both sides
]


def dev():
    return torch.device("cuda", 0)


def run_all(layer, case, bn, training):
    F = torch.tensor(case["F"], device=dev())
    W = torch.tensor(case["W"], device=dev())
    gO = torch.tensor(case["gO"], device=dev())
    stds = torch.tensor(case["stds"], device=dev()) if bn else None
    flags = (1 if bn else 0) | (2 if training else 0)
    FF = layer.product_fwd(F)
    O = layer.mix_fwd(FF, W, stds, 2.0, 1e-5, flags)
    gFF, gW = layer.mix_bwd(gO, FF, W, stds, 2.0, 1e-5, flags)
    gF = layer.product_bwd(F, gFF)
    torch.cuda.synchronize()
    return dict(CG=layer.CG, FF=FF, O=O, gFF=gFF, gW=gW, gF=gF, stds=stds)


@pytest.mark.parametrize("bn,training", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("taus,tau_out,B,mode", CASES)
def test_drop_in_module_against_reference_extension(taus, tau_out, B, mode, bn, training):
    from cgnet_b200 import CG_cuda_ops as shim
    from cgnet_b200 import _lib, get_plan
    assert shim.sparse_maxL() == 511
    case = make_case(taus, tau_out, B, mode, seed=61)
    ours = run_all(refdrv.RefLayer.from_case(shim, case, dev()), case, bn, training)

    # the library's own module path on the same inputs: same kernels, so the same bits
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev())
    F = torch.tensor(case["F"], device=dev())
    W = torch.tensor(case["W"], device=dev())
    stds = torch.tensor(case["stds"], device=dev()) if bn else None
    flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if training else 0)
    FF = plan.cg_product_fwd(F)
    O = plan.fn_wmm_fwd(FF, W, stds, 2.0, 1e-5, flags)
    assert torch.equal(FF, ours["FF"]) and torch.equal(O, ours["O"])
    if bn:
        assert torch.equal(stds, ours["stds"])

    if not refdrv.available():
        pytest.skip("reference CUDA extension not built: compared with the library's own path only")
    if 0 in taus or 0 in tau_out:
        return   # empty fragments are this library's edge case; the reference's kernels are not run on shapes its own test never uses
    ref = run_all(refdrv.RefLayer.from_case(refdrv.load_ops(), case, dev()), case, bn, training)
    t_ff = case["t_ff"]
    np.testing.assert_allclose(ours["CG"].cpu().numpy(), ref["CG"].cpu().numpy(), atol=3e-7, rtol=0)
    assert_fragments_close(ours["FF"].cpu().numpy(), ref["FF"].cpu().numpy(), t_ff, "FF")
    assert_fragments_close(ours["O"].cpu().numpy(), ref["O"].cpu().numpy(), tau_out, "O")
    assert_fragments_close(ours["gFF"].cpu().numpy(), ref["gFF"].cpu().numpy(), t_ff, "gFF")
    assert_weights_close(ours["gW"].cpu().numpy(), ref["gW"].cpu().numpy(), t_ff, tau_out, "gW")
    assert_fragments_close(ours["gF"].cpu().numpy(), ref["gF"].cpu().numpy(), taus, "gF")
    if training:
        np.testing.assert_allclose(ours["stds"].cpu().numpy(), ref["stds"].cpu().numpy(), rtol=2e-5, atol=1e-7)


def test_drop_in_module_checks_its_arguments():
    from cgnet_b200 import CG_cuda_ops as shim
    case = make_case([2, 2, 2], [2, 2, 2], 2, "default", seed=62)
    layer = refdrv.RefLayer.from_case(shim, case, dev())
    F = torch.tensor(case["F"], device=dev())
    with pytest.raises(RuntimeError, match="shape"):
        layer.product_fwd(F[:, :-1].contiguous())          # activation of the wrong length: refused, not read out of bounds
    with pytest.raises(RuntimeError, match="float32"):
        layer.product_fwd(F.double())
    FF = layer.product_fwd(F)
    W = torch.tensor(case["W"], device=dev())
    with pytest.raises(RuntimeError, match="shape"):
        layer.mix_fwd(FF, W[:-1].contiguous(), None, 1.0, 1e-5, 0)
