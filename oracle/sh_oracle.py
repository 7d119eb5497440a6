"""CPU restatement of the reference's spherical-harmonic projection (utils/s2_sph.py, utils/geometries.py).

TEST INFRASTRUCTURE ONLY (imported by tests/ and bench.py's CPU leg; nothing under cgnet_b200/ imports it).

The reference takes its sample grid, quadrature weights and spherical harmonics from the third-party package
`lie_learn` (imports at utils/s2_sph.py:5-7; no version pinned in the reference's README, and the package is absent
here), so those three pieces are restated from the package's published definitions:
  * `lie_learn.spaces.S2.meshgrid(b, 'Gauss-Legendre')`: colatitudes arccos of the b+1 Gauss-Legendre nodes, longitudes
    k pi / (b+1) for k < 2b+2, 'ij' order;
  * `S2.quadrature_weights(b, 'Gauss-Legendre')`: node weight times 2 pi / (2b+2) (they sum to 4 pi);
  * `spherical_harmonics.csh(l, m, theta, phi, 'quantum', True)`: orthonormal Y_lm with the Condon-Shortley phase,
    evaluated here through scipy.special (an independent implementation of the same convention).
PARITY UNPINNED for these third-party pieces: the reference repository holds no fixture of them and the package cannot
be run here.  What the reference itself computes with them is restated line by line and is what the parity tests hold
the CUDA path to:  coefs = ((fs * ws)[:, None] * conj(sphs)).mean(0) * 4 pi   (utils/s2_sph.py:84-85)
                   coefs = (f[:, None] * sph).mean(0) * 4 pi                    (utils/geometries.py:142).
"""
import numpy as np
from numpy.polynomial.legendre import leggauss


def csh(l, m, theta, phi):
    """Y_lm(theta = colatitude, phi = longitude), 'quantum' normalisation, Condon-Shortley phase."""
    import scipy.special as sp
    if hasattr(sp, "sph_harm_y"):
        return sp.sph_harm_y(l, m, theta, phi)
    return sp.sph_harm(m, l, phi, theta)


def grid_and_weights(b):
    """theta, phi, ws of `get_grid_and_weights(b, 'Gauss-Legendre')` (utils/s2_sph.py:20-26): flattened, phi shifted by -pi."""
    x, w = leggauss(b + 1)
    beta = np.arccos(x)
    alpha = np.arange(2 * b + 2) * np.pi / (b + 1)
    theta, phi = np.meshgrid(beta, alpha, indexing="ij")
    ws = w[:, None] * (2 * np.pi / (2 * b + 2) * np.ones(2 * b + 2)[None, :])
    return theta.flatten(), phi.flatten() - np.pi, ws.flatten()


def default_sphs(lmax):
    """`get_default_sphs(lmax)` (utils/s2_sph.py:32-39): (points, lmax^2) for l < lmax on the bandwidth-lmax grid."""
    theta, phi, _ = grid_and_weights(lmax)
    sph = np.zeros((len(theta), lmax ** 2), dtype=complex)
    for l in range(lmax):
        for m in range(-l, l + 1):
            sph[:, l ** 2 + (m + l)] = csh(l, m, theta, phi)
    return sph


def get_sph_coefs_on_grid(fs, lmax):
    """`get_sph_coefs` (utils/s2_sph.py:79-86) for values already sampled on the grid (its resampling step, an
    interpolation of scattered data, is not part of the contraction)."""
    _, _, ws = grid_and_weights(lmax)
    sphs = default_sphs(lmax)
    coefs = (np.expand_dims(fs * ws, 1) * np.conj(sphs)).mean(0)
    return coefs * 4 * np.pi


def get_coef_C(f, beta, alpha, lmax):
    """`get_coef_C` (utils/geometries.py:125-144): scattered points, (lmax+1)^2 columns, no weights, no conjugate."""
    sph = np.zeros((len(f), (lmax + 1) ** 2), dtype=complex)
    for l in range(lmax + 1):
        for m in range(-l, l + 1):
            sph[:, l ** 2 + (m + l)] = csh(l, m, beta, alpha)
    coefs = (np.expand_dims(f, 1) * sph).mean(0) * 4 * np.pi
    return coefs, sph
