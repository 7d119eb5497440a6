"""Mesh -> sphere projection of the SHREC17 front end on the GPU (reference: ``Shrec17/dataset.py:40-95,146-182``).

``make_sgrid`` / ``render_model`` / ``ProjectOnSphere`` keep the reference's names and results; the mesh is passed as
arrays (vertices ``(V, 3)``, faces ``(F, 3)``) instead of a trimesh object, because the ray casting is done by
libcgnet_b200.so (``cgb200_raycast_sphere``: brute-force Moeller-Trumbore in double precision, deterministic first
hit) and not by trimesh.  Face normals follow the winding of the faces as given (the reference repairs the winding
with trimesh's ``fix_normals`` when it loads a mesh, ``dataset.py:114``); the convex hull is wound outwards here.
Loading and cleaning mesh files stays outside this module.
"""
import numpy as np
import torch

from . import _lib

__all__ = ["rotmat", "make_sgrid", "render_model", "ProjectOnSphere"]

# per-channel (mean, std) the reference subtracts and divides by (dataset.py:167-178)
NORMALISATION = [(0.75, 0.26), (0.59, 0.50), (0.54, 0.29), (0.52, 0.19), (0.80, 0.18), (0.51, 0.25)]


def rotmat(a, b, c, hom_coord=False):
    """ZYZ-Euler rotation matrix, optionally homogeneous (``dataset.py:15-37``)."""
    def z(t):
        return np.array([[np.cos(t), np.sin(t), 0, 0], [-np.sin(t), np.cos(t), 0, 0], [0, 0, 1, 0], [0, 0, 0, 1]])

    def y(t):
        return np.array([[np.cos(t), 0, np.sin(t), 0], [0, 1, 0, 0], [-np.sin(t), 0, np.cos(t), 0], [0, 0, 0, 1]])
    r = z(a).dot(y(b)).dot(z(c))
    return r if hom_coord else r[:3, :3]


def make_sgrid(b, alpha=0.0, beta=0.0, gamma=0.0):
    """The 'SOFT' grid of bandwidth ``b`` (colatitudes pi(2j+1)/(4b), longitudes 2 pi k/(2b), ``(2b)**2`` points) as
    Cartesian points on the unit sphere, rotated by the ZYZ angles (``dataset.py:40-50``)."""
    th = np.pi * (2 * np.arange(2 * b) + 1) / (4.0 * b)
    ph = np.arange(2 * b) * np.pi / b
    theta, phi = np.meshgrid(th, ph, indexing="ij")
    sgrid = np.stack([np.sin(theta) * np.cos(phi), np.sin(theta) * np.sin(phi), np.cos(theta)], -1).reshape(-1, 3)
    return np.einsum("ij,nj->ni", rotmat(alpha, beta, gamma), sgrid)


def render_model(vertices, faces, sgrid, device="cuda"):
    """``(3, points)`` float32 CUDA tensor: distance to the first hit of the inward ray from every grid point (1 where
    it meets nothing), n . g and |n ^ g| of the hit triangle (0 where none) (``dataset.py:53-95``)."""
    lib = _lib.load()
    dev = torch.device(device)
    if dev.type != "cuda":
        raise RuntimeError("render_model runs on a CUDA device (cgnet_b200 has no CPU path)")
    if dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())

    def as_dev(x, dtype, cols):
        t = x if isinstance(x, torch.Tensor) else torch.as_tensor(np.ascontiguousarray(x))
        t = t.to(device=dev, dtype=dtype).contiguous()
        if t.dim() != 2 or t.shape[1] != cols:
            raise RuntimeError(f"expected an (N, {cols}) array, got {tuple(t.shape)}")
        return t
    v = as_dev(vertices, torch.float32, 3)
    f = as_dev(faces, torch.int32, 3)
    g = as_dev(sgrid, torch.float32, 3)
    image = torch.empty(3, g.shape[0], dtype=torch.float32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    n = int(lib.cgb200_raycast_workspace_bytes(f.shape[0]))
    if n < 0:
        _lib.check(1, "cgb200_raycast_workspace_bytes")
    ws = torch.empty(max(n, 256), dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        _lib.check(lib.cgb200_raycast_sphere(v.data_ptr(), v.shape[0], f.data_ptr(), f.shape[0], g.data_ptr(), g.shape[0],
                                             image.data_ptr(), ws.data_ptr(), n, status.data_ptr(),
                                             torch.cuda.current_stream(dev).cuda_stream), "cgb200_raycast_sphere")
    if int(status.item()) != 0:
        raise RuntimeError("the cgnet_b200 ray-casting kernel gave up on a bounded wait")
    return image


def _convex_hull(vertices):
    from scipy.spatial import ConvexHull
    v = np.asarray(vertices, dtype=np.float64)
    hull = ConvexHull(v)
    faces = hull.simplices.copy()
    n = np.cross(v[faces[:, 1]] - v[faces[:, 0]], v[faces[:, 2]] - v[faces[:, 0]])
    flip = (n * hull.equations[:, :3]).sum(1) < 0
    faces[flip] = faces[flip][:, ::-1]
    return v, faces


class ProjectOnSphere:
    """``ProjectOnSphere(bandwidth)(vertices, faces)`` -> ``(6, 2b, 2b)`` float32 CUDA tensor: the three channels of the
    mesh and of its convex hull, normalised per channel (``dataset.py:146-182``)."""

    def __init__(self, bandwidth, device="cuda"):
        self.bandwidth = bandwidth
        self.device = device
        self.sgrid = make_sgrid(bandwidth, alpha=0, beta=0, gamma=0)
        self._norm = None

    def __call__(self, vertices, faces):
        im = render_model(vertices, faces, self.sgrid, self.device)
        try:
            hv, hf = _convex_hull(vertices.cpu().numpy() if isinstance(vertices, torch.Tensor) else vertices)
        except Exception:   # degenerate hull: the reference falls back to the mesh itself (dataset.py:155-159)
            hv, hf = vertices, faces
        hull_im = render_model(hv, hf, self.sgrid, self.device)
        im = torch.cat([im, hull_im], 0)
        if self._norm is None or self._norm.device != im.device:
            self._norm = torch.tensor(NORMALISATION, dtype=torch.float32, device=im.device)
        im = (im - self._norm[:, :1]) / self._norm[:, 1:]
        return im.reshape(6, 2 * self.bandwidth, 2 * self.bandwidth)

    def __repr__(self):
        return self.__class__.__name__ + "(bandwidth={0})".format(self.bandwidth)
