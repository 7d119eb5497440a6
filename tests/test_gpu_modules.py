"""The PyTorch module surface on a GPU: SphericalCNN / SphericalCNN_fast against a layer-by-layer oracle composition,
list and flat calling conventions, state-dict compatibility with the reference's key names, persistence of the norm
counter, randomly drawn shapes, and rotation invariance of the network's output."""
import numpy as np
import pytest
import torch

import cg_oracle as o
from helpers import TOL, make_case, oracle_layer, rel_fro

pytestmark = pytest.mark.gpu


def dev():
    return torch.device("cuda", 0)


def oracle_network(x, taus, Ws, stds_list, lmax, llls, training):
    """Embedding of the reference's SphericalCNN.forward (CGNet/CGNet.py:52-69) with the oracle's layers, fp64."""
    B = x.shape[0]
    fs = o.split_fragments(x, taus[0])
    emb = [fs[0].reshape(B, -1)]
    new_stds = []
    for i in range(len(taus) - 1):
        fs, ns = o.cgbn_layer(fs, taus[i], taus[i + 1], lmax, llls, Ws[i], stds=stds_list[i], cnt=1.0, training=training)
        new_stds.append(ns)
        emb.append(fs[0].reshape(B, -1))
    return torch.cat(emb, 1), new_stds


@pytest.mark.parametrize("training", [False, True])
@pytest.mark.parametrize("sparse", [False, True])
def test_spherical_cnn_matches_oracle_network(training, sparse):
    from cgnet_b200 import SphericalCNN
    lmax, taus, B = 4, [[1] * 5, [3, 2, 2, 1, 1], [2] * 5, [4, 1, 1, 1, 1]], 6
    torch.manual_seed(3)
    net = SphericalCNN(lmax, taus, sparse_flag=sparse, device=dev())
    net.train(training)
    assert net.output_length == 2 * (1 + 3 + 2 + 4)
    assert [k for k in net.state_dict() if k.startswith("cgs.0.")] == ["cgs.0.bnWMM.bn_eps", "cgs.0.bnWMM.bn_stds", "cgs.0.bnWMM.W",
                                                                        "cgs.0.bnWMM.bn_cnt_buf"]
    llls = list(net.cgs[0].cg.lll_list)
    rng = np.random.RandomState(0)
    x_np = rng.randn(B, 25, 2).astype(np.float32)
    Ws = [torch.tensor(c.bnWMM.W.detach().cpu().numpy(), dtype=torch.float64, requires_grad=True) for c in net.cgs]
    stds = [c.bnWMM.bn_stds.detach().cpu().numpy().copy() for c in net.cgs]
    xo = torch.tensor(x_np, dtype=torch.float64, requires_grad=True)
    want, new_stds = oracle_network(xo, taus, Ws, stds, lmax, llls, training)
    g = torch.tensor(rng.randn(*want.shape))
    (want * g).sum().backward()

    x = torch.tensor(x_np, device=dev(), requires_grad=True)
    got = net(x)
    (got * g.to(dev(), torch.float32)).sum().backward()
    assert rel_fro(got.detach().cpu().numpy(), want.detach().numpy()) < TOL
    assert rel_fro(x.grad.cpu().numpy(), xo.grad.numpy()) < TOL
    for c, W in zip(net.cgs, Ws):
        assert rel_fro(c.bnWMM.W.grad.cpu().numpy(), W.grad.numpy()) < TOL
    if training:
        for c, s in zip(net.cgs, new_stds):
            np.testing.assert_allclose(c.bnWMM.bn_stds.detach().cpu().numpy(), s, rtol=5e-5, atol=1e-6)
            assert c.bnWMM.bn_cnt == 2.0
    # the list calling convention gives the same embedding
    net.eval()
    with torch.no_grad():
        a = net(x.detach())
        b = net([f.contiguous() for f in o.split_fragments(x.detach(), taus[0])])
    assert torch.equal(a, b)


def test_layer_list_and_flat_outputs_and_state_dict_round_trip():
    from cgnet_b200 import CGBN_cuda
    lmax, taus, tau_out = 3, [2, 3, 1, 2], [3, 1, 2, 2]
    a = CGBN_cuda(lmax, taus, tau_out, device=dev())
    x = torch.randn(4, sum(t * (2 * l + 1) for l, t in enumerate(taus)), 2, device=dev())
    a.train()
    for _ in range(3):
        a(x)
    assert a.bnWMM.bn_cnt == 4.0
    flat = a(x, straight_output=True)
    a.eval()
    frs = a([f.contiguous() for f in o.split_fragments(x, taus)])
    assert [tuple(f.shape) for f in frs] == [(4, t, 2 * l + 1, 2) for l, t in enumerate(tau_out)]
    b = CGBN_cuda(lmax, taus, tau_out, device=dev())
    b.load_state_dict(a.state_dict())
    assert b.bnWMM.bn_cnt == a.bnWMM.bn_cnt                     # the reference loses this counter on resume
    b.eval()
    assert torch.equal(torch.cat([f.reshape(4, -1, 2) for f in frs], 1), b(x, straight_output=True))
    # a checkpoint written by the reference has no counter entry: it must still load
    sd = {k: v for k, v in a.state_dict().items() if "bn_cnt" not in k}
    c = CGBN_cuda(lmax, taus, tau_out, device=dev())
    c.load_state_dict(sd)
    assert c.bnWMM.bn_cnt == 1.0
    assert flat.shape == (4, sum(t * (2 * l + 1) for l, t in enumerate(tau_out)), 2)


def test_spherical_cnn_fast_front_end():
    from cgnet_b200 import SphericalCNN, SphericalCNN_fast
    lmax, C, B = 3, 2, 5
    torch.manual_seed(5)
    fast = SphericalCNN_fast(lmax, [3] * 4, 2, skip_type=1, num_channels_input=C, device=dev())
    assert fast.output_length == 2 * (C + 3 + 3)
    rng = np.random.RandomState(1)
    coeffs = (rng.randn(B, C, (lmax + 1) ** 2) + 1j * rng.randn(B, C, (lmax + 1) ** 2)).astype(np.complex64)
    flat = fast.pack(coeffs)
    # fragment l, channel c, order m holds coefficient l*l + l + m of input function c
    off = 0
    for l in range(lmax + 1):
        blk = flat[:, off:off + C * (2 * l + 1)].reshape(B, C, 2 * l + 1, 2).cpu().numpy()
        np.testing.assert_allclose(blk[..., 0] + 1j * blk[..., 1], coeffs[:, :, l * l:(l + 1) ** 2], rtol=1e-6)
        off += C * (2 * l + 1)
    plain = SphericalCNN(lmax, [[C] * 4, [3] * 4, [3] * 4], device=dev())
    plain.load_state_dict(fast.state_dict())
    fast.eval(), plain.eval()
    with torch.no_grad():
        assert torch.equal(fast(coeffs), plain(flat))


@pytest.mark.parametrize("seed", range(12))
def test_random_shapes_against_oracle(seed):
    """Randomly drawn (lmax, channel counts, batch, pair list, norm mode): fused layer vs oracle."""
    from cgnet_b200 import _lib, get_plan
    rng = np.random.RandomState(1000 + seed)
    lmax = int(rng.randint(0, 7))
    taus = [int(rng.randint(0 if lmax > 1 else 1, 7)) for _ in range(lmax + 1)]
    if sum(taus) == 0:
        taus[0] = 1
    tau_out = [int(rng.randint(1, 9)) for _ in range(lmax + 1)]
    B = int(rng.choice([1, 2, 31, 32, 33, 65]))
    mode = ["default", "mst", "debug"][int(rng.randint(0, 3))]
    bn, training = bool(rng.randint(0, 2)), bool(rng.randint(0, 2))
    case = make_case(taus, tau_out, B, mode, seed=seed)
    plan = get_plan(lmax, taus, tau_out, case["llls"], dev())
    O_want, gF_want, gW_want, stds_want = oracle_layer(case, bn, training and bn, cnt=1.0)
    t = lambda a: torch.tensor(a, device=dev())
    stds = t(case["stds"]) if bn else None
    flags = (_lib.FN_PRESENT if bn else 0) | (_lib.FN_UPDATE if (training and bn) else 0)
    O = plan.layer_fwd(t(case["F"]), t(case["W"]), stds, 1.0, 1e-5, flags)
    gF, gW = plan.layer_bwd(t(case["F"]), t(case["W"]), stds, 1e-5, flags & 1, t(case["gO"]))
    what = f"lmax={lmax} taus={taus} tau_out={tau_out} B={B} {mode} bn={bn} train={training}"
    assert rel_fro(O.cpu().numpy(), O_want) < TOL, what
    assert rel_fro(gF.cpu().numpy(), gF_want) < TOL or np.linalg.norm(gF_want) == 0, what
    assert rel_fro(gW.cpu().numpy(), gW_want) < TOL or np.linalg.norm(gW_want) == 0, what


def _wigner_d_small(l, beta):
    """Wigner small-d matrix d^l_{m'm}(beta), indices m', m = -l..l (standard closed-form sum)."""
    from math import factorial as f
    d = np.zeros((2 * l + 1, 2 * l + 1))
    for mp in range(-l, l + 1):
        for m in range(-l, l + 1):
            s = 0.0
            for k in range(max(0, m - mp), min(l + m, l - mp) + 1):
                s += ((-1) ** (k - m + mp) * np.cos(beta / 2) ** (2 * l - 2 * k + m - mp) * np.sin(beta / 2) ** (2 * k - m + mp)
                      / (f(l + m - k) * f(k) * f(mp - m + k) * f(l - mp - k)))
            d[mp + l, m + l] = np.sqrt(f(l + mp) * f(l - mp) * f(l + m) * f(l - m)) * s
    return d


def test_network_output_is_rotation_invariant():
    """Rotating the input function (every degree-l fragment multiplied by the Wigner matrix D^l) must not change the
    l = 0 outputs of a CG network: the property the architecture exists for, independent of any reference output."""
    from cgnet_b200 import SphericalCNN
    lmax, B = 4, 3
    taus = [[2] * 5, [3] * 5, [2] * 5]
    torch.manual_seed(9)
    net = SphericalCNN(lmax, taus, device=dev())
    net.eval()
    rng = np.random.RandomState(4)
    x = rng.randn(B, sum(2 * (2 * l + 1) for l in range(lmax + 1)), 2)
    alpha, beta, gamma = 0.7, 1.1, -0.4
    xr = np.zeros_like(x)
    off = 0
    for l in range(lmax + 1):
        n = 2 * l + 1
        m = np.arange(-l, l + 1)
        D = np.exp(-1j * alpha * m)[:, None] * _wigner_d_small(l, beta) * np.exp(-1j * gamma * m)[None, :]
        blk = x[:, off:off + 2 * n].reshape(B, 2, n, 2)
        z = blk[..., 0] + 1j * blk[..., 1]
        zr = np.einsum("pm,btm->btp", D, z)
        xr[:, off:off + 2 * n] = np.stack([zr.real, zr.imag], -1).reshape(B, 2 * n, 2)
        off += 2 * n
    with torch.no_grad():
        a = net(torch.tensor(x, dtype=torch.float32, device=dev())).cpu().numpy()
        b = net(torch.tensor(xr, dtype=torch.float32, device=dev())).cpu().numpy()
    assert rel_fro(b, a) < 2e-4
