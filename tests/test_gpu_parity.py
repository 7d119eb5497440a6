"""Parity of the CUDA path against the CPU oracle and the committed reference fixtures.  Every call goes through the
C ABI of libcgnet_b200.so.  Tolerance: relative Frobenius error per fragment < 1e-4 in fp32 (helpers.TOL); index and
size results must be exact."""
import numpy as np
import pytest
import torch

import cg_oracle as o
from helpers import (TOL, assert_fragments_close, assert_weights_close, make_case, oracle_layer, oracle_product, rel_fro)

pytestmark = pytest.mark.gpu

SHAPES = [
    # taus, tau_out, B, pair mode
    ([2, 1], [2, 1], 2, "mst"),                       # the reference test's default invocation (CGNet/test.py:130)
    ([3, 2, 1, 1, 1], [3, 2, 1, 1, 1], 1, "default"),  # CGNet/test.py:81
    ([2, 1, 1], [2, 1, 1], 2, "default"),
    ([2, 2, 2, 2], [3, 1, 2, 2], 3, "debug"),
    ([4] * 6, [4] * 6, 3, "default"),
    ([3, 1, 4, 1, 5, 2, 2], [2, 3, 1, 4, 1, 2, 3], 2, "mst"),
    ([1], [3], 5, "default"),                          # lmax = 0
    ([5] * 4, [5] * 4, 37, "default"),                 # batch not a multiple of the warp size
    ([1] * 6, [5] * 6, 33, "default"),                 # single input channel per degree (first layer of the MNIST net)
    ([8] * 6, [8] * 6, 32, "default"),                 # the reference's CPU-runnable case: lmax 5, 8 channels, batch 32
    ([6, 0, 3, 2], [2, 2, 0, 3], 4, "default"),        # empty fragments on both sides
    ([7, 6, 5], [20, 3, 17], 3, "default"),            # more than 16 output channels, ragged tiles
    ([2] * 21, [2] * 21, 5, "mst"),                    # lmax = 20: fragments of 41 rows
]


def dev():
    return torch.device("cuda", 0)


def plan_for(case):
    from cgnet_b200 import get_plan
    return get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev(), depthwise=case["depthwise"])


def t(x):
    return torch.tensor(x, device=dev())


def test_library_and_device():
    from cgnet_b200 import _lib
    lib = _lib.load()
    assert lib.cgb200_version() >= 100
    assert torch.cuda.get_device_capability(0)[0] >= 10, "these kernels are built for sm_100a only"


@pytest.mark.parametrize("lmax,mode", [(3, "default"), (6, "default"), (10, "default"), (6, "mst"), (20, "mst"), (30, "default")])
def test_cg_table_matches_oracle(lmax, mode):
    from cgnet_b200.cg_layers import _precomputeCG_cuda
    from helpers import ltuples
    llls, _ = o.encode_sorted(ltuples(mode, lmax))
    if lmax == 30:
        llls = llls[::37] + llls[-5:]
        llls = sorted(llls)
    cg, offs = _precomputeCG_cuda(lmax, llls, dev())
    want, want_offs = o.cg_band_table(lmax, llls)
    np.testing.assert_array_equal(offs.cpu().numpy(), want_offs)
    np.testing.assert_allclose(cg.cpu().numpy(), want, atol=3e-7, rtol=0)


def test_cg_table_matches_reference_fixture(golden_cg):
    from cgnet_b200.cg_layers import _precomputeCG_cuda
    for L in (3, 6):
        llls, _ = o.encode_sorted(o.default_ltuples(L))
        cg, _ = _precomputeCG_cuda(L, llls, dev())
        np.testing.assert_allclose(cg.cpu().numpy(), golden_cg[f"band_default_{L}"], atol=3e-7, rtol=0)


@pytest.mark.parametrize("taus,tau_out,B,mode", SHAPES)
def test_product_forward_backward(taus, tau_out, B, mode):
    case = make_case(taus, tau_out, B, mode, seed=11)
    plan = plan_for(case)
    assert plan.t_ff() == [int(x) for x in case["t_ff"]]
    ff_want, gf_want = oracle_product(case)
    F = t(case["F"])
    FF = plan.cg_product_fwd(F)
    assert_fragments_close(FF.cpu().numpy(), ff_want, case["t_ff"], "FF")
    gF = plan.cg_product_bwd(F, t(case["gFF"]))
    assert_fragments_close(gF.cpu().numpy(), gf_want, taus, "gF (product)")


@pytest.mark.parametrize("bn,training", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("taus,tau_out,B,mode", SHAPES)
def test_two_pass_layer(taus, tau_out, B, mode, bn, training):
    from cgnet_b200 import _lib
    case = make_case(taus, tau_out, B, mode, seed=12)
    plan = plan_for(case)
    O_want, gF_want, gW_want, stds_want = oracle_layer(case, bn, training, cnt=3.0)
    F, W = t(case["F"]), t(case["W"])
    stds = t(case["stds"]) if bn else None
    flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if training else 0)
    FF = plan.cg_product_fwd(F)
    O = plan.fn_wmm_fwd(FF, W, stds, 3.0, 1e-5, flags)
    assert_fragments_close(O.cpu().numpy(), O_want, tau_out, "O")
    if training:
        np.testing.assert_allclose(stds.cpu().numpy(), stds_want, rtol=2e-5, atol=1e-7)
    gFF, gW = plan.fn_wmm_bwd(t(case["gO"]), FF, W, stds, 1e-5, flags & _lib.FN_PRESENT)
    assert_weights_close(gW.cpu().numpy(), gW_want, case["t_ff"], tau_out, "gW")
    gF = plan.cg_product_bwd(F, gFF)
    assert_fragments_close(gF.cpu().numpy(), gF_want, taus, "gF")


@pytest.mark.parametrize("bn,training", [(False, False), (True, False), (True, True)])
@pytest.mark.parametrize("taus,tau_out,B,mode", SHAPES)
def test_fused_layer(taus, tau_out, B, mode, bn, training):
    from cgnet_b200 import _lib
    case = make_case(taus, tau_out, B, mode, seed=13)
    plan = plan_for(case)
    O_want, gF_want, gW_want, stds_want = oracle_layer(case, bn, training, cnt=2.0)
    F, W = t(case["F"]), t(case["W"])
    stds = t(case["stds"]) if bn else None
    flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if training else 0)
    O = plan.layer_fwd(F, W, stds, 2.0, 1e-5, flags)
    assert_fragments_close(O.cpu().numpy(), O_want, tau_out, "O (fused)")
    if training:
        np.testing.assert_allclose(stds.cpu().numpy(), stds_want, rtol=2e-5, atol=1e-7)
    gF, gW = plan.layer_bwd(F, W, stds, 1e-5, flags & _lib.FN_PRESENT, t(case["gO"]))
    assert_weights_close(gW.cpu().numpy(), gW_want, case["t_ff"], tau_out, "gW (fused)")
    assert_fragments_close(gF.cpu().numpy(), gF_want, taus, "gF (fused)")


@pytest.mark.parametrize("taus,tau_out,B", [([3] * 4, [3] * 4, 5), ([4, 4, 4], [2, 5, 3], 40), ([6] * 3, [7] * 3, 3)])
def test_depthwise_extension(taus, tau_out, B):
    """Channel-wise product (t1 == t2): no reference counterpart, checked against the oracle's restatement only."""
    from cgnet_b200 import _lib
    for mode in ("default", "mst"):
        case = make_case(taus, tau_out, B, mode, seed=14, depthwise=True)
        plan = plan_for(case)
        ff_want, gf_want = oracle_product(case)
        F, W, stds = t(case["F"]), t(case["W"]), t(case["stds"])
        FF = plan.cg_product_fwd(F)
        assert_fragments_close(FF.cpu().numpy(), ff_want, case["t_ff"], "FF (depthwise)")
        assert_fragments_close(plan.cg_product_bwd(F, t(case["gFF"])).cpu().numpy(), gf_want, taus, "gF (depthwise product)")
        O_want, gF_want, gW_want, stds_want = oracle_layer(case, True, True, cnt=1.0)
        flags = _lib.FN_PRESENT | _lib.FN_UPDATE
        O = plan.layer_fwd(F, W, stds, 1.0, 1e-5, flags)
        assert_fragments_close(O.cpu().numpy(), O_want, tau_out, "O (depthwise fused)")
        np.testing.assert_allclose(stds.cpu().numpy(), stds_want, rtol=2e-5, atol=1e-7)
        gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, t(case["gO"]))
        assert_weights_close(gW.cpu().numpy(), gW_want, case["t_ff"], tau_out, "gW (depthwise fused)")
        assert_fragments_close(gF.cpu().numpy(), gF_want, taus, "gF (depthwise fused)")


LAYER_CASES = ["t21_mst", "t21_default", "t32111_default", "t32111_mst", "t211_default", "t2222_debug",
               "L5t4_default", "L6ragged_mst"]


@pytest.mark.parametrize("fused", [False, True])
@pytest.mark.parametrize("name", LAYER_CASES)
def test_against_reference_fixtures(golden_layers, name, fused):
    """Outputs and gradients of the reference's own Python path (tests/golden/layer_cases.npz), through the modules."""
    from cgnet_b200 import CGBN_cuda, CG_woFilter_cuda
    g = {k.split("/", 1)[1]: golden_layers[k] for k in golden_layers.files if k.startswith(name + "/")}
    taus, tau_out, llls = g["taus"].tolist(), g["tau_out"].tolist(), g["llls"].tolist()
    L = len(taus) - 1
    mode = name.split("_")[1]
    lll_mode = {"default": None, "mst": "mst", "debug": "debug"}[mode]
    t_ff, _ = o.tau_ff_and_offsets(L, taus, llls)

    cg = CG_woFilter_cuda(L, taus, lll_mode=lll_mode, device=dev())
    assert list(cg.lll_list) == llls and [int(x) for x in cg.t_FF] == t_ff.tolist()
    F = t(g["F"]).requires_grad_(True)
    FF = cg(F)
    if "FF" in g:
        assert_fragments_close(FF.detach().cpu().numpy(), g["FF"], t_ff, "FF vs reference twin")
        g_ff = t(g["gFF"])
    else:
        g_ff = torch.tensor(np.random.RandomState(1234).randn(*FF.shape), dtype=torch.float, device=dev())
        norms = [float(f.norm()) for f in o.split_fragments(FF.detach().cpu(), t_ff)]
        np.testing.assert_allclose(norms, g["FF_fragnorm"], rtol=1e-4)
    (FF * g_ff).sum().backward()
    assert_fragments_close(F.grad.cpu().numpy(), g["cg_gF"], taus, "product gF vs reference twin")

    for key, bn, training in (("nobn", False, False), ("bneval", True, False), ("harness_bntrain", True, True)):
        layer = CGBN_cuda(L, taus, tau_out, batchnorm=bn, sparse_flag=(mode == "mst"), device=dev(), fused=fused,
                          lll_mode=lll_mode)
        with torch.no_grad():
            layer.bnWMM.W.copy_(t(g["W"]))
            if bn:
                layer.bnWMM.bn_stds.copy_(t(g["stds"]))
        layer.train(training)
        F = t(g["F"]).requires_grad_(True)
        O = layer(F, straight_output=True)
        assert_fragments_close(O.detach().cpu().numpy(), g[f"{key}_O"], tau_out, f"{key} O vs reference twin")
        (O * t(g["gO"])).sum().backward()
        assert_fragments_close(F.grad.cpu().numpy(), g[f"{key}_gF"], taus, f"{key} gF vs reference twin")
        assert_weights_close(layer.bnWMM.W.grad.cpu().numpy(), g[f"{key}_gW"], t_ff, tau_out, f"{key} gW vs reference twin")
        if training:
            # the twin takes np.std of an fp32 array; the CUDA path (like the reference's) accumulates in double
            np.testing.assert_allclose(layer.bnWMM.bn_stds.detach().cpu().numpy(), g["harness_bntrain_stds"], rtol=3e-5, atol=1e-6)
            assert layer.bnWMM.bn_cnt == 2.0


def test_runs_are_bit_identical():
    from cgnet_b200 import _lib
    case = make_case([5] * 5, [5] * 5, 50, "default", seed=15)
    plan = plan_for(case)
    F, W, gO = t(case["F"]), t(case["W"]), t(case["gO"])
    outs = []
    for _ in range(2):
        stds = t(case["stds"])
        O = plan.layer_fwd(F, W, stds, 1.0, 1e-5, _lib.FN_PRESENT | _lib.FN_UPDATE)
        gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
        FF = plan.cg_product_fwd(F)
        gFF, gW2 = plan.fn_wmm_bwd(gO, FF, W, stds, 1e-5, _lib.FN_PRESENT)
        outs.append([x.cpu().numpy().copy() for x in (O, gF, gW, stds, FF, gFF, gW2)])
    for a, b in zip(*outs):
        assert np.array_equal(a, b)


def test_empty_batch_and_bad_arguments():
    from cgnet_b200 import CGBN_cuda, _lib
    case = make_case([2, 2, 2], [2, 2, 2], 0, "default", seed=16)
    plan = plan_for(case)
    F = t(case["F"])
    assert plan.cg_product_fwd(F).shape == (0, plan.n_FF, 2)
    O = plan.layer_fwd(F, t(case["W"]), None, 1.0, 1e-5, 0)
    assert O.shape == (0, plan.n_O, 2)
    gF, gW = plan.layer_bwd(F, t(case["W"]), None, 1e-5, 0, t(case["gO"]))
    assert float(gW.abs().sum()) == 0.0
    layer = CGBN_cuda(2, [2, 2, 2], [2, 2, 2], device=dev())
    with pytest.raises(RuntimeError, match="CUDA tensor"):
        layer(torch.zeros(1, 18, 2))
    with pytest.raises(RuntimeError, match="float32"):
        layer(torch.zeros(1, 18, 2, device=dev(), dtype=torch.float64))
    # a workspace that is too small is refused with a message, not a fault
    lib = _lib.load()
    one = make_case([2, 2, 2], [2, 2, 2], 4, "default", seed=16)
    ws = torch.empty(256, dtype=torch.uint8, device=dev())
    Od = torch.empty(4, plan.n_O, 2, device=dev())
    rc = lib.cgb200_layer_fwd(plan.handle, t(one["F"]).data_ptr(), t(one["W"]).data_ptr(), None, 1.0, 1e-5, 0, Od.data_ptr(), 4,
                              ws.data_ptr(), 256, None)
    assert rc == 4 and b"workspace" in lib.cgb200_last_error()


def test_input_gradient_is_optional():
    """A layer whose input needs no gradient (the first layer of a network) skips that part of the backward."""
    from cgnet_b200 import CGBN_cuda, _lib
    case = make_case([1] * 5, [4] * 5, 9, "default", seed=17)
    plan = plan_for(case)
    F, W, gO = t(case["F"]), t(case["W"]), t(case["gO"])
    gF_full, gW_full = plan.layer_bwd(F, W, None, 1e-5, 0, gO)
    gF_none, gW_only = plan.layer_bwd(F, W, None, 1e-5, 0, gO, need_gF=False)
    assert gF_none is None and torch.equal(gW_full, gW_only)
    layer = CGBN_cuda(4, [1] * 5, [4] * 5, batchnorm=False, device=dev())
    with torch.no_grad():
        layer.bnWMM.W.copy_(W)
    O = layer(F, straight_output=True)          # F does not require grad
    (O * gO).sum().backward()
    assert torch.equal(layer.bnWMM.W.grad, gW_full)


def test_layer_runs_inside_a_cuda_graph():
    """Forward and backward captured into one CUDA graph (the backward forks its weight gradient onto a second stream
    and joins it back inside the call, which a capture must be able to follow) and replayed on new inputs."""
    from cgnet_b200 import _lib
    case = make_case([5] * 6, [5] * 6, 40, "default", seed=16)
    other = make_case([5] * 6, [5] * 6, 40, "default", seed=17)
    plan = plan_for(case)
    F, W, gO, stds = t(case["F"]), t(case["W"]), t(case["gO"]), t(case["stds"])
    flags = _lib.FN_PRESENT
    plan.layer_fwd(F, W, stds, 1.0, 1e-5, flags)          # first calls outside the capture: lazy set-up happens here
    plan.layer_bwd(F, W, stds, 1e-5, flags, gO)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        O = plan.layer_fwd(F, W, stds, 1.0, 1e-5, flags)
        gF, gW = plan.layer_bwd(F, W, stds, 1e-5, flags, gO)
    for src in (other, case):
        F.copy_(t(src["F"]))
        gO.copy_(t(src["gO"]))
        graph.replay()
        torch.cuda.synchronize()
        got = [x.cpu().numpy().copy() for x in (O, gF, gW)]
        O2 = plan.layer_fwd(F, W, stds, 1.0, 1e-5, flags)
        gF2, gW2 = plan.layer_bwd(F, W, stds, 1e-5, flags, gO)
        torch.cuda.synchronize()
        for a, b in zip(got, (O2, gF2, gW2)):
            assert np.array_equal(a, b.cpu().numpy())


@pytest.mark.parametrize("taus,tau_out,B", [([3, 2, 2], [2, 3, 1], 4800), ([5] * 3, [5] * 3, 4770)])
def test_more_sample_groups_than_sms(taus, tau_out, B):
    """A batch of more than 148 x 32 samples: more sample groups than SMs, so the forward leaves its persistent
    shared-memory variant for the row-per-block one, and every kernel's group loops and group slices run long."""
    from cgnet_b200 import _lib
    case = make_case(taus, tau_out, B, "default", seed=18)
    plan = plan_for(case)
    O_want, gF_want, gW_want, stds_want = oracle_layer(case, True, True, cnt=3.0)
    F, W, gO, stds = t(case["F"]), t(case["W"]), t(case["gO"]), t(case["stds"])
    O = plan.layer_fwd(F, W, stds, 3.0, 1e-5, _lib.FN_PRESENT | _lib.FN_UPDATE)
    gF, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
    torch.cuda.synchronize()
    assert_fragments_close(O.cpu().numpy(), O_want, tau_out, "O, large batch")
    assert_fragments_close(gF.cpu().numpy(), gF_want, taus, "gF, large batch")
    assert_weights_close(gW.cpu().numpy(), gW_want, case["t_ff"], tau_out, "gW, large batch")
    np.testing.assert_allclose(stds.cpu().numpy(), stds_want, rtol=2e-5, atol=1e-7)
