"""The tensor-core (tcgen05 + tensor memory + bulk async copy, 3xTF32) variant of the fused forward against the CPU
oracle and against the CUDA-core variant.  Tolerance as everywhere: relative Frobenius error per fragment < 1e-4."""
import contextlib

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


@contextlib.contextmanager
def option(plan, opt, value):
    """Select a kernel variant through the plan's options for the duration of a block (plans are shared, so the
    library's default is restored afterwards)."""
    from cgnet_b200 import _lib
    plan.set_option(opt, value)
    try:
        yield
    finally:
        plan.set_option(opt, _lib.AUTO)


def _forward(plan, case, bn, training, tc):
    from cgnet_b200 import _lib
    dev = torch.device("cuda", 0)
    with option(plan, _lib.OPT_TC_FWD, 1 if tc else 0):
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if training else 0)
        O = plan.layer_fwd(F, W, stds, 2.0, 1e-5, flags)
        plan.check_status()   # raises if a bounded wait inside the tensor-core kernel ran out
        return O.cpu().numpy(), None if stds is None else stds.cpu().numpy()


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
    with option(plan, _lib.OPT_TC_GRAD_W, 1 if tc else 0):
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        _, gW = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT if bn else 0, gO)
        plan.check_status()
        return gW.cpu().numpy()


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
    with option(plan, _lib.OPT_TC_GRAD_F, 1 if tc else 0):
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        gF, _ = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT if bn else 0, gO)
        plan.check_status()
        return gF.cpu().numpy()


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


def test_bounded_wait_gives_up_cleanly():
    """The give-up path of the tensor-core kernels, driven without a fault, a trap or an endless loop: with the test
    option that keeps the MMA warp idle nothing ever arrives at the barriers the other warps wait on, so their waits run
    out after a short iteration limit.  The kernel must then return by itself, report through the plan's status word,
    mark the outputs it owns with NaN, and leave the context usable: the same call with the options restored gives the
    right answer."""
    from cgnet_b200 import _lib, get_plan
    dev = torch.device("cuda", 0)
    case = make_case([4] * 3, [16] * 3, 5, "default", seed=57)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev)
    assert plan.tile == 4
    F = torch.tensor(case["F"], device=dev)
    W = torch.tensor(case["W"], device=dev)
    gO = torch.tensor(case["gO"], device=dev)
    plan.set_option(_lib.OPT_WAIT_POLLS, 2000)
    plan.set_option(_lib.OPT_TEST_IDLE_MMA, 1)
    plan.set_option(_lib.OPT_TC_STAGES, 2)   # fewer stages than cells: the producers' waits run out too, not only the epilogue's
    try:
        with option(plan, _lib.OPT_TC_FWD, 1):
            O_bad = plan.layer_fwd(F, W, None, 1.0, 1e-5, 0)
        with pytest.raises(RuntimeError, match="gave up"):
            plan.check_status()
        assert torch.isnan(O_bad).all(), "a forward that gave up must mark every output it owns"
        with option(plan, _lib.OPT_TC_GRAD_W, 1), option(plan, _lib.OPT_GRAD_MID_GEMM, 1):
            gF_bad, gW_bad = plan.layer_bwd(F, W, None, 1e-5, 0, gO)
        with pytest.raises(RuntimeError, match="gave up"):
            plan.check_status()
        assert torch.isnan(gW_bad).all()
        assert torch.isnan(gF_bad).all(), "the mid-gradient GEMM marks its tiles, so every input gradient built on them is NaN"
    finally:
        plan.set_option(_lib.OPT_TEST_IDLE_MMA, _lib.AUTO)
        plan.set_option(_lib.OPT_WAIT_POLLS, _lib.AUTO)
        plan.set_option(_lib.OPT_TC_STAGES, _lib.AUTO)
    plan.check_status()   # the word was cleared by the reads above
    O_want, _, gW_want, _ = oracle_layer(case, False, False)
    O_good, _ = _forward(plan, case, False, False, tc=True)
    assert_fragments_close(O_good, O_want, case["tau_out"], "O after a run that gave up")
    import cg_oracle as o
    t_ff, _ = o.tau_ff_and_offsets(case["lmax"], case["taus"], case["llls"])
    assert_weights_close(_weight_gradient(plan, case, False, tc=True), gW_want, t_ff, case["tau_out"], "gW after a run that gave up")


def test_unsupported_variant_is_refused():
    """Forcing a tensor-core variant on a plan without its tables is an error at the option call, not a silent fallback."""
    from cgnet_b200 import _lib, get_plan
    case = make_case([5] * 3, [5] * 3, 2, "default", seed=58)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], torch.device("cuda", 0))
    assert plan.tile == 5
    with pytest.raises(RuntimeError, match="no tables"):
        plan.set_option(_lib.OPT_TC_FWD, 1)


@pytest.mark.parametrize("staged", [1, 2])
@pytest.mark.parametrize("taus,tau_out,B,mode", [([8] * 4, [16] * 4, 40, "default"), ([16] * 6, [16] * 6, 33, "default"),
                                                 ([8] * 11, [32] * 11, 20, "default"), ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default")])
def test_staged_tensor_core_forward_equals_unstaged(taus, tau_out, B, mode, staged):
    """The opt-in forward whose staging warp bulk-copies each cell's band rows, operand rows and weights into a
    shared-memory ring (1) or the band rows and weights only (2): same arithmetic in the same order as the default
    tensor-core forward, so the same bits."""
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, mode, seed=59)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    assert plan.tile == 4
    with option(plan, _lib.OPT_TC_FWD_SPLIT, 0):   # the staged kernel never splits the contraction
        want, _ = _forward(plan, case, True, False, tc=True)
    with option(plan, _lib.OPT_TC_STAGED, staged):
        got, _ = _forward(plan, case, True, False, tc=True)
    assert np.array_equal(got, want)


@pytest.mark.parametrize("taus,tau_out,B,mode", [([8] * 4, [16] * 4, 40, "default"), ([16] * 6, [16] * 6, 33, "default"),
                                                 ([8] * 11, [32] * 11, 20, "default"), ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default"),
                                                 ([2] * 5, [8] * 5, 3, "default")])
def test_split_contraction_of_tensor_core_forward(taus, tau_out, B, mode):
    """Every splitting level of the tensor-core forward (the degree with the most cells cut into 1, 2, 4, ... 64 parts of
    its cells, partial outputs added in part order) against the oracle; the level the launch would pick by itself is one
    of them, and each level is deterministic."""
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, mode, seed=60)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    assert plan.tile in (2, 4)
    O_want, _, _, _ = oracle_layer(case, True, False, cnt=2.0)
    auto, _ = _forward(plan, case, True, False, tc=True)
    hits = 0
    for level in range(7):
        with option(plan, _lib.OPT_TC_FWD_SPLIT, level):
            got, _ = _forward(plan, case, True, False, tc=True)
            again, _ = _forward(plan, case, True, False, tc=True)
        assert np.array_equal(got, again), f"level {level} is not deterministic"
        assert_fragments_close(got, O_want, tau_out, f"O (tensor-core forward, splitting level {level}) vs oracle")
        hits += int(np.array_equal(got, auto))
    assert hits >= 1


def _input_gradient_gemm(plan, case, bn, gemm):
    from cgnet_b200 import _lib
    dev = torch.device("cuda", 0)
    with option(plan, _lib.OPT_GRAD_MID_GEMM, int(gemm)):   # 0 off, 1 on, 2 / 3 on with two / one block per SM forced
        F = torch.tensor(case["F"], device=dev)
        W = torch.tensor(case["W"], device=dev)
        gO = torch.tensor(case["gO"], device=dev)
        stds = torch.tensor(case["stds"], device=dev) if bn else None
        gF, _ = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT if bn else 0, gO)
        plan.check_status()
        return gF.cpu().numpy()


@pytest.mark.parametrize("bn", [False, True])
@pytest.mark.parametrize("taus,tau_out,B,mode", [([8] * 4, [16] * 4, 40, "default"), ([16] * 6, [16] * 6, 33, "default"),
                                                 ([8] * 11, [32] * 11, 20, "default"), ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default"),
                                                 ([8] * 8, [12] * 8, 64, "mst"), ([8] * 3, [64] * 3, 3, "default"),
                                                 ([6, 0, 8, 4], [8, 4, 0, 20], 4, "default"),
                                                 ([4] * 16, [12] * 16, 3, "mst"), ([4] * 21, [12] * 21, 2, "mst")])
def test_input_gradient_through_mid_gradient_gemm(taus, tau_out, B, mode, bn):
    """The input gradient whose first phase is a tensor-core GEMM into the workspace (the gradient of the mid activation,
    every tile once, in the layout the gather kernel keeps it in shared memory) against the oracle and against the kernel
    that rebuilds the tiles on the CUDA cores; ragged channel counts, empty fragments on both sides, every group size of
    the GEMM (4, 2 and 1 cells per group at 16, 32 and 64 output channels); lmax 15 and 20, where the gather kernel cannot
    hold a whole tile beside two staging buffers and reads it in chunks."""
    from cgnet_b200 import get_plan
    case = make_case(taus, tau_out, B, mode, seed=61)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0), tile=4)
    _, gF_want, _, _ = oracle_layer(case, bn, False)
    got = _input_gradient_gemm(plan, case, bn, gemm=True)
    again = _input_gradient_gemm(plan, case, bn, gemm=True)
    assert np.array_equal(got, again), "not deterministic"
    assert_fragments_close(got, gF_want, taus, "gF (mid-gradient GEMM) vs oracle")
    assert_fragments_close(got, _input_gradient_gemm(plan, case, bn, gemm=False), taus, "gF (mid-gradient GEMM) vs CUDA-core tiles")
    # the gather kernel as one block per SM with the whole tile resident, and as two blocks per SM with the tile in chunks
    for forced in (2, 3):
        one = _input_gradient_gemm(plan, case, bn, gemm=forced)
        assert np.array_equal(one, _input_gradient_gemm(plan, case, bn, gemm=forced)), "not deterministic"
        assert_fragments_close(one, gF_want, taus, f"gF (mid-gradient GEMM, gather variant {forced}) vs oracle")


@pytest.mark.parametrize("taus,tau_out,B,mode", [([8] * 4, [16] * 4, 40, "default"), ([16] * 6, [16] * 6, 33, "default"),
                                                 ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default"), ([6, 0, 8, 4], [8, 4, 0, 20], 4, "default"),
                                                 ([8] * 8, [12] * 8, 64, "mst")])
def test_forward_reads_back_the_tiles_the_statistics_kernel_kept(taus, tau_out, B, mode):
    """Forward with a statistics update on the tensor-core path: the statistics kernel keeps the tiles of the mid
    activation it generates and the forward kernel loads them instead of generating them again.  Both run the same
    generator, so output and updated statistics must be the same bits as with the variant switched off, and both must
    match the oracle."""
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, mode, seed=62)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0), tile=4)
    O_want, _, _, stds_want = oracle_layer(case, True, True, cnt=2.0)
    out = {}
    for keep in (0, 1):
        with option(plan, _lib.OPT_FWD_KEEP_MID, keep):
            out[keep] = _forward(plan, case, True, True, tc=True)
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    assert_fragments_close(out[1][0], O_want, tau_out, "O (tiles kept by the statistics kernel) vs oracle")
    np.testing.assert_allclose(out[1][1], stds_want, rtol=2e-5, atol=1e-7)


@pytest.mark.parametrize("taus,tau_out,B,mode", [([8] * 4, [16] * 4, 40, "default"), ([16] * 6, [16] * 6, 33, "default"),
                                                 ([8, 4, 12, 8], [6, 9, 16, 3], 7, "default"), ([6, 0, 8, 4], [8, 4, 0, 20], 4, "default")])
def test_backward_reads_the_tiles_kept_in_the_forwards_workspace(taus, tau_out, B, mode):
    """A forward with a statistics update leaves the mid activation's tiles at the start of its workspace; handed the same
    workspace (CGB200_FN_KEEP_MID), the backward's weight gradient loads them instead of generating them again.  Same
    generator, so the gradients are the same bits as those of a backward with a fresh workspace; both match the oracle."""
    from cgnet_b200 import _lib, get_plan
    import cg_oracle as o
    dev = torch.device("cuda", 0)
    case = make_case(taus, tau_out, B, mode, seed=63)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], dev, tile=4)
    assert plan.keeps_mid(B)
    F = torch.tensor(case["F"], device=dev)
    W = torch.tensor(case["W"], device=dev)
    gO = torch.tensor(case["gO"], device=dev)
    stds = torch.tensor(case["stds"], device=dev)
    O, ws = plan.layer_fwd(F, W, stds, 2.0, 1e-5, _lib.FN_PRESENT | _lib.FN_UPDATE, keep=True)
    gF_k, gW_k = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO, kept=ws)
    gF_n, gW_n = plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
    plan.check_status()
    assert torch.equal(gW_k, gW_n) and torch.equal(gF_k, gF_n)
    O_want, gF_want, gW_want, _ = oracle_layer(case, True, True, cnt=2.0)
    assert_fragments_close(O.cpu().numpy(), O_want, tau_out, "O")
    assert_fragments_close(gF_k.cpu().numpy(), gF_want, taus, "gF with the kept workspace")
    t_ff, _ = o.tau_ff_and_offsets(case["lmax"], case["taus"], case["llls"])
    assert_weights_close(gW_k.cpu().numpy(), gW_want, t_ff, tau_out, "gW from the kept tiles")


def test_module_keeps_the_workspace_between_forward_and_backward():
    """CGBN_cuda in training: with keep_mid the layer's workspace travels from the forward to the backward; parameters'
    and input's gradients are the same bits as without."""
    from cgnet_b200 import CGBN_cuda
    dev = torch.device("cuda", 0)
    grads = {}
    for keep in (False, True):
        torch.manual_seed(5)
        np.random.seed(5)
        layer = CGBN_cuda(4, [16] * 5, [16] * 5, batchnorm=True, device=dev, keep_mid=keep).train()
        assert layer.cg.plan.tile == 4
        torch.manual_seed(6)
        x = torch.randn(37, 16 * 25, 2, device=dev, requires_grad=True)
        out = layer(x, straight_output=True)
        assert layer._keeps_mid(37) == keep
        (out * torch.linspace(-1, 1, out.numel(), device=dev).reshape(out.shape)).sum().backward()
        grads[keep] = (x.grad.clone(), layer.bnWMM.W.grad.clone(), layer.bnWMM.bn_stds.detach().clone())
        layer.cg.plan.check_status()
    for a, b in zip(grads[False], grads[True]):
        assert torch.equal(a, b)


@pytest.mark.parametrize("taus,tau_out,B,mode", [([5] * 6, [5] * 6, 37, "default"), ([8] * 4, [8] * 4, 40, "default"),
                                                 ([6, 0, 3, 5], [2, 7, 0, 3], 4, "default"), ([10] * 5, [5] * 5, 70, "mst")])
def test_cuda_core_forward_reads_back_the_kept_tiles(taus, tau_out, B, mode):
    """The same on the CUDA-core forward (under 12 output channels: the benchmark network's layers; the statistics kernel
    of tile edges 5 and 6 stores its tile in two halves): identical bits with the variant on and off, and the oracle's
    values."""
    from cgnet_b200 import _lib, get_plan
    case = make_case(taus, tau_out, B, mode, seed=64)
    plan = get_plan(case["lmax"], taus, tau_out, case["llls"], torch.device("cuda", 0))
    O_want, _, _, stds_want = oracle_layer(case, True, True, cnt=2.0)
    out = {}
    for keep in (0, 1):   # forced on also where the default leaves it off (tile edge 3 in the ragged case)
        with option(plan, _lib.OPT_FWD_KEEP_MID, keep):
            out[keep] = _forward(plan, case, True, True, tc=False)
    assert np.array_equal(out[0][0], out[1][0]) and np.array_equal(out[0][1], out[1][1])
    assert_fragments_close(out[1][0], O_want, tau_out, "O (CUDA-core forward, kept tiles) vs oracle")
    np.testing.assert_allclose(out[1][1], stds_want, rtol=2e-5, atol=1e-7)


def test_inference_with_weights_packed_once():
    """cgb200_layer_pack_weights + cgb200_layer_fwd_packed against cgb200_layer_fwd (same bits), and the module-level cache:
    CGBN_cuda in eval mode under no_grad packs once, notices new weights, new statistics and a training step in between."""
    from cgnet_b200 import CGBN_cuda, _lib, get_plan
    dev = torch.device("cuda", 0)
    case = make_case([8, 4, 12, 8], [6, 9, 16, 3], 7, "default", seed=65)
    plan = get_plan(case["lmax"], case["taus"], case["tau_out"], case["llls"], dev, tile=4)
    assert plan.packed_weights_bytes() > 0
    F = torch.tensor(case["F"], device=dev)
    W = torch.tensor(case["W"], device=dev)
    stds = torch.tensor(case["stds"], device=dev)
    for fl, st in ((_lib.FN_PRESENT, stds), (0, None)):
        want = plan.layer_fwd(F, W, st, 1.0, 1e-5, fl)
        got = plan.layer_fwd_packed(F, plan.pack_weights(W, st, 1e-5, fl))
        plan.check_status()
        assert torch.equal(got, want)
    narrow = get_plan(2, [5] * 3, [5] * 3, make_case([5] * 3, [5] * 3, 2, "default", seed=1)["llls"], dev)
    assert narrow.packed_weights_bytes() == 0        # CUDA-core forward: nothing to pack

    torch.manual_seed(7)
    np.random.seed(7)
    layer = CGBN_cuda(3, [16] * 4, [16] * 4, batchnorm=True, device=dev)
    x = torch.randn(9, 16 * 16, 2, device=dev)

    def both():
        layer.eval()
        with torch.no_grad():
            cached = layer(x, straight_output=True)
        plain = layer(x, straight_output=True)       # autograd on: the ordinary call, packs inside
        assert torch.equal(cached, plain)
        return cached

    a = both()
    key = layer._packed_key
    assert key is not None and torch.equal(both(), a) and layer._packed_key == key      # second call: cache hit
    with torch.no_grad():
        layer.bnWMM.W.mul_(1.5)
    b = both()
    assert layer._packed_key != key and not torch.equal(a, b)
    layer.train()
    layer(x, straight_output=True)                   # updates the statistics in place (no tensor version changes)
    c = both()
    assert not torch.equal(b, c)
