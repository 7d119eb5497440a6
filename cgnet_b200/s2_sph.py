"""Spherical-harmonic projection of sampled functions on the GPU: the step in front of the CG network.

Mirrors the two projection routines of the reference's preprocessing,

    get_sph_coefs(fs, lmax)                utils/s2_sph.py:79-86     values on the Gauss-Legendre grid of bandwidth lmax
    get_coef_C(f, beta, alpha, lmax)       utils/geometries.py:125-144   values at scattered points

which compute, one function at a time in numpy, ``((f * w)[:, None] * conj(Y)).mean(0) * 4 pi`` resp.
``(f[:, None] * Y).mean(0) * 4 pi``.  Here a `SHProjector` evaluates the basis once on the host (grid, weights and
harmonics restated below: the reference takes them from the `lie_learn` package), packs it on the device, and projects a
whole batch of functions with one tensor-core GEMM in libcgnet_b200.so (`cgb200_sh_project`).  There is no CPU path for
the contraction.
"""
import numpy as np
import torch
from numpy.polynomial.legendre import leggauss

from . import _lib

__all__ = ["gauss_legendre_grid", "spherical_harmonics", "SHProjector", "get_sph_coefs", "get_coef_C"]


def gauss_legendre_grid(b):
    """Colatitudes, longitudes and quadrature weights of the Gauss-Legendre grid of bandwidth ``b``, flattened, as the
    reference's ``get_grid_and_weights`` returns them (``utils/s2_sph.py:20-26``): b+1 Gauss nodes in colatitude times
    2b+2 equally spaced longitudes shifted by -pi; weights = node weight times 2 pi / (2b+2) (they sum to 4 pi)."""
    x, w = leggauss(b + 1)
    beta = np.arccos(x)
    alpha = np.arange(2 * b + 2) * np.pi / (b + 1)
    theta, phi = np.meshgrid(beta, alpha, indexing="ij")
    ws = np.repeat(w[:, None] * (2 * np.pi / (2 * b + 2)), 2 * b + 2, axis=1)
    return theta.reshape(-1), phi.reshape(-1) - np.pi, ws.reshape(-1)


def spherical_harmonics(n_degrees, theta, phi):
    """Orthonormal complex spherical harmonics with the Condon-Shortley phase (what the reference calls
    ``csh(l, m, theta, phi, 'quantum', True)``) for l < ``n_degrees`` at colatitudes ``theta`` and longitudes ``phi``:
    a complex128 array ``(points, n_degrees**2)`` with (l, m) in column ``l*l + l + m``.

    Evaluated with the standard three-term recurrence on the fully normalised associated Legendre functions (stable to
    degrees far beyond what the network uses), vectorised over the points."""
    theta = np.asarray(theta, dtype=np.float64).reshape(-1)
    phi = np.asarray(phi, dtype=np.float64).reshape(-1)
    L = int(n_degrees)
    out = np.zeros((theta.size, L * L), dtype=np.complex128)
    if L == 0:
        return out
    ct, st = np.cos(theta), np.sin(theta)
    pmm = np.full(theta.size, np.sqrt(1.0 / (4.0 * np.pi)))          # normalised P_m^m, starting at m = 0
    for m in range(L):
        if m > 0:
            pmm = -np.sqrt((2.0 * m + 1.0) / (2.0 * m)) * st * pmm   # Condon-Shortley phase in the sign
        e = np.exp(1j * m * phi)
        p_prev2, p_prev = None, pmm
        for l in range(m, L):
            if l == m:
                p = pmm
            elif l == m + 1:
                p = np.sqrt(2.0 * m + 3.0) * ct * pmm
            else:
                a = np.sqrt((4.0 * l * l - 1.0) / (l * l - m * m))
                b = np.sqrt(((l - 1.0) ** 2 - m * m) / (4.0 * (l - 1.0) ** 2 - 1.0))
                p = a * (ct * p_prev - b * p_prev2)
            if l > m:
                p_prev2, p_prev = p_prev, p
            y = p * e
            out[:, l * l + l + m] = y
            if m > 0:
                out[:, l * l + l - m] = (-1) ** m * np.conj(y)
    return out


class SHProjector:
    """Projection onto ``n_degrees**2`` harmonics for a fixed set of sample points, on one CUDA device.

    ``weights`` (per point) and ``conjugate`` select the two forms of the reference: ``conjugate=True`` with the grid's
    quadrature weights is ``get_sph_coefs``; ``conjugate=False`` without weights is ``get_coef_C``.  ``project(f)`` takes
    real samples ``(..., points)`` (any leading shape, float32 CUDA tensor) and returns ``(..., n_degrees**2, 2)``.
    """

    def __init__(self, n_degrees, theta, phi, weights=None, conjugate=True, device="cuda"):
        lib = _lib.load()
        self.device = torch.device(device)
        if self.device.type != "cuda":
            raise RuntimeError("SHProjector lives on a CUDA device (cgnet_b200 has no CPU path)")
        if self.device.index is None:
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.n_degrees = int(n_degrees)
        self.n_cols = self.n_degrees ** 2
        sph = spherical_harmonics(self.n_degrees, theta, phi)
        self.sph = sph                                    # as the reference hands back from get_coef_C
        basis = np.conj(sph) if conjugate else sph
        if weights is not None:
            basis = basis * np.asarray(weights, dtype=np.float64).reshape(-1, 1)
        self.n_points = basis.shape[0]
        self.scale = float(4.0 * np.pi / self.n_points)   # `.mean(0) * 4 pi`
        b = torch.tensor(np.stack([basis.real, basis.imag], -1).astype(np.float32), device=self.device).contiguous()
        nbytes = int(lib.cgb200_sh_basis_bytes(self.n_points, self.n_cols))
        if nbytes < 0:
            _lib.check(1, "cgb200_sh_basis_bytes")
        self._packed = torch.empty(nbytes, dtype=torch.uint8, device=self.device)
        self._status = torch.zeros(1, dtype=torch.int32, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(lib.cgb200_sh_basis_pack(b.data_ptr(), self.n_points, self.n_cols, self._packed.data_ptr(),
                                                torch.cuda.current_stream(self.device).cuda_stream), "cgb200_sh_basis_pack")
        torch.cuda.current_stream(self.device).synchronize()   # `b` may be freed once the pack kernel has read it

    def project(self, f):
        if not isinstance(f, torch.Tensor) or f.device != self.device or f.dtype != torch.float32:
            raise RuntimeError(f"samples must be a float32 tensor on {self.device}")
        if f.shape[-1] != self.n_points:
            raise RuntimeError(f"samples have {f.shape[-1]} points, the projector {self.n_points}")
        lead = f.shape[:-1]
        f2 = f.reshape(-1, self.n_points).contiguous()
        rows = f2.shape[0]
        lib = _lib.load()
        out = torch.empty(rows, self.n_cols, 2, dtype=torch.float32, device=self.device)
        n = int(lib.cgb200_sh_workspace_bytes(rows, self.n_points))
        ws = torch.empty(max(n, 256), dtype=torch.uint8, device=self.device)
        with torch.cuda.device(self.device):
            _lib.check(lib.cgb200_sh_project(f2.data_ptr(), rows, self.n_points, self.n_cols, self._packed.data_ptr(), self.scale,
                                             out.data_ptr(), ws.data_ptr(), n, self._status.data_ptr(),
                                             torch.cuda.current_stream(self.device).cuda_stream), "cgb200_sh_project")
        return out.reshape(*lead, self.n_cols, 2)

    def check_status(self):
        """Raise if the projection kernel gave up on a bounded device-side wait since the last check (synchronises)."""
        if int(self._status.item()) != 0:
            self._status.zero_()
            raise RuntimeError("the cgnet_b200 projection kernel gave up on a bounded wait; the coefficients of that call are NaN")


_grid_projectors = {}


def get_sph_coefs(fs, lmax, device=None):
    """Coefficients (l < ``lmax``) of functions sampled on the Gauss-Legendre grid of bandwidth ``lmax``
    (``utils/s2_sph.py:79-86`` without its resampling step): ``fs`` is ``(..., (lmax+1)(2 lmax+2))`` float32 on a CUDA
    device, the result ``(..., lmax**2, 2)``."""
    dev = fs.device if device is None else torch.device(device)
    key = (int(lmax), str(dev))
    if key not in _grid_projectors:
        theta, phi, ws = gauss_legendre_grid(int(lmax))
        _grid_projectors[key] = SHProjector(int(lmax), theta, phi, weights=ws, conjugate=True, device=dev)
    return _grid_projectors[key].project(fs)


def get_coef_C(f, beta, alpha, lmax=14, sph=None):
    """``(coefs, projector)`` for values ``f`` ``(..., points)`` at colatitudes ``beta`` and longitudes ``alpha``
    (``utils/geometries.py:125-144``, complex harmonics): ``(lmax+1)**2`` columns, no weights, no conjugate.  As in the
    reference the second result can be passed back as ``sph`` to reuse the basis for the next call."""
    proj = sph if isinstance(sph, SHProjector) else SHProjector(int(lmax) + 1, beta, alpha, weights=None, conjugate=False, device=f.device)
    return proj.project(f), proj
