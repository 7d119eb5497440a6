"""Spherical-harmonic projection (the step in front of the network): host evaluator against scipy on CPU, and the
tensor-core contraction against the CPU restatement of the reference's two routines on the GPU.  Tolerance of the GPU
tests: relative Frobenius error < 1e-4 (fp32 against fp64)."""
import numpy as np
import pytest
import torch

import sh_oracle
from helpers import TOL, rel_fro


def test_host_harmonics_match_scipy():
    from cgnet_b200.s2_sph import spherical_harmonics
    rng = np.random.RandomState(0)
    theta = np.concatenate([[0.0, np.pi, 1e-9], rng.uniform(0, np.pi, 50)])     # poles included
    phi = np.concatenate([[0.0, 1.0, -2.0], rng.uniform(-np.pi, np.pi, 50)])
    L = 31
    got = spherical_harmonics(L, theta, phi)
    for l in (0, 1, 2, 5, 14, 30):
        for m in range(-l, l + 1):
            np.testing.assert_allclose(got[:, l * l + l + m], sh_oracle.csh(l, m, theta, phi), atol=2e-12, rtol=0)


def test_grid_matches_restatement_and_is_a_quadrature():
    from cgnet_b200.s2_sph import gauss_legendre_grid, spherical_harmonics
    for b in (3, 10, 14):
        theta, phi, ws = gauss_legendre_grid(b)
        t2, p2, w2 = sh_oracle.grid_and_weights(b)
        np.testing.assert_array_equal(theta, t2)
        np.testing.assert_array_equal(phi, p2)
        np.testing.assert_allclose(ws, w2, rtol=1e-15)
        assert len(theta) == (b + 1) * (2 * b + 2) and abs(ws.sum() - 4 * np.pi) < 1e-12
        Y = spherical_harmonics(b, theta, phi)
        gram = (Y.conj() * ws[:, None]).T @ Y           # exact for products of degree < 2b + 2
        np.testing.assert_allclose(gram, np.eye(b * b), atol=1e-12)


@pytest.mark.gpu
@pytest.mark.parametrize("lmax,batch", [(10, 37), (14, 130), (3, 1)])
def test_grid_projection_matches_reference_formula(lmax, batch):
    from cgnet_b200.s2_sph import get_sph_coefs
    dev = torch.device("cuda", 0)
    n = (lmax + 1) * (2 * lmax + 2)
    rng = np.random.RandomState(lmax)
    fs = rng.randn(batch, n).astype(np.float32)
    got = get_sph_coefs(torch.tensor(fs, device=dev), lmax).cpu().numpy()
    want = np.stack([sh_oracle.get_sph_coefs_on_grid(fs[i].astype(np.float64), lmax) for i in range(batch)])
    assert got.shape == (batch, lmax * lmax, 2)
    assert rel_fro(got[..., 0] + 1j * got[..., 1], want) < TOL
    # a band-limited function comes back as its own coefficients times the reference's 4 pi / points factor
    c = (rng.randn(lmax * lmax) + 1j * rng.randn(lmax * lmax))
    for l in range(lmax):                                   # make the function real: c_{l,-m} = (-1)^m conj(c_{l,m})
        for m in range(1, l + 1):
            c[l * l + l - m] = (-1) ** m * np.conj(c[l * l + l + m])
        c[l * l + l] = c[l * l + l].real
    f = (sh_oracle.default_sphs(lmax) @ c).real.astype(np.float32)
    back = get_sph_coefs(torch.tensor(f[None], device=dev), lmax).cpu().numpy()[0]
    np.testing.assert_allclose(back[:, 0] + 1j * back[:, 1], c * 4 * np.pi / n, atol=2e-5 * np.abs(c).max())


@pytest.mark.gpu
@pytest.mark.parametrize("lmax,points,batch,channels", [(14, 4096, 3, 6), (5, 100, 2, 1), (20, 1000, 2, 2)])
def test_scattered_projection_matches_reference_formula(lmax, points, batch, channels):
    """`get_coef_C` on scattered points, with the basis reused for a second call as the reference's `sph=` argument does
    (lmax 14, six channels, 64 x 64 points is the shape of the reference's SHREC17 preprocessing; lmax 20 needs two
    column tiles, 1000 points a ragged last chunk)."""
    from cgnet_b200.s2_sph import get_coef_C
    dev = torch.device("cuda", 0)
    rng = np.random.RandomState(points)
    beta = rng.uniform(0, np.pi, points)
    alpha = rng.uniform(0, 2 * np.pi, points)
    f = rng.randn(batch, channels, points).astype(np.float32)
    got, proj = get_coef_C(torch.tensor(f, device=dev), beta, alpha, lmax=lmax)
    assert got.shape == (batch, channels, (lmax + 1) ** 2, 2)
    want = np.stack([[sh_oracle.get_coef_C(f[b, c].astype(np.float64), beta, alpha, lmax)[0] for c in range(channels)] for b in range(batch)])
    g = got.cpu().numpy()
    assert rel_fro(g[..., 0] + 1j * g[..., 1], want) < TOL
    again, proj2 = get_coef_C(torch.tensor(f[:1], device=dev), beta, alpha, lmax=lmax, sph=proj)
    assert proj2 is proj and torch.equal(again, got[:1])
    proj.check_status()


@pytest.mark.gpu
def test_long_quadrature_keeps_its_accuracy():
    """128 x 128 sample points: 6144 tensor-core accumulation steps per output, summed in rounded pieces."""
    from cgnet_b200.s2_sph import SHProjector
    dev = torch.device("cuda", 0)
    rng = np.random.RandomState(9)
    P, L = 16384, 15
    beta, alpha = rng.uniform(0, np.pi, P), rng.uniform(0, 2 * np.pi, P)
    proj = SHProjector(L, beta, alpha, conjugate=False, device=dev)
    f = (1.0 + rng.rand(200, P)).astype(np.float32)            # all positive: partial sums grow steadily, the hard case for truncation
    got = proj.project(torch.tensor(f, device=dev)).cpu().numpy()
    want = (f.astype(np.float64) @ proj.sph) * (4 * np.pi / P)
    err = rel_fro(got[..., 0] + 1j * got[..., 1], want)
    print(f"\n[parity] projection over {P} points: {err:.2e}")
    assert err < TOL
    proj.check_status()
