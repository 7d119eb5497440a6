"""CPU restatement of the reference's mesh -> sphere rendering (Shrec17/dataset.py:40-95,146-182).

TEST INFRASTRUCTURE ONLY.  The reference takes the ray / triangle intersections from the third-party package `trimesh`
(`mesh.ray.intersects_id(..., multiple_hits=False)`, dataset.py:57-58; version unpinned, package absent here) and the
grid from `lie_learn.spaces.S2` ('SOFT' grid).  Both are restated from their published definitions: the first
intersection of a ray with a triangle soup by the Moeller-Trumbore test in float64, the SOFT grid as colatitudes
pi (2j+1) / (4b) and longitudes 2 pi k / (2b).  PARITY UNPINNED for those third-party pieces; everything the reference
itself computes from the hits (distance, n . g, |n ^ g|, channel normalisation) is restated line by line.
"""
import numpy as np


def rotmat(a, b, c):
    """ZYZ Euler rotation (dataset.py:15-37)."""
    def z(t):
        return np.array([[np.cos(t), np.sin(t), 0], [-np.sin(t), np.cos(t), 0], [0, 0, 1]])

    def y(t):
        return np.array([[np.cos(t), 0, np.sin(t)], [0, 1, 0], [-np.sin(t), 0, np.cos(t)]])
    return z(a).dot(y(b)).dot(z(c))


def make_sgrid(b, alpha=0.0, beta=0.0, gamma=0.0):
    """dataset.py:40-50: SOFT grid of bandwidth b as Cartesian points on the unit sphere, rotated."""
    th = np.pi * (2 * np.arange(2 * b) + 1) / (4.0 * b)
    ph = np.arange(2 * b) * np.pi / b
    theta, phi = np.meshgrid(th, ph, indexing="ij")
    sgrid = np.stack([np.sin(theta) * np.cos(phi), np.sin(theta) * np.sin(phi), np.cos(theta)], -1).reshape(-1, 3)
    return np.einsum("ij,nj->ni", rotmat(alpha, beta, gamma), sgrid)


def first_hits(vertices, faces, origins, directions, chunk=256):
    """Index of the first triangle each ray meets (-1: none) and the ray parameter of the hit."""
    v = np.asarray(vertices, dtype=np.float64)
    f = np.asarray(faces, dtype=np.int64)
    v0, e1, e2 = v[f[:, 0]], v[f[:, 1]] - v[f[:, 0]], v[f[:, 2]] - v[f[:, 0]]
    best_f = np.full(len(origins), -1, dtype=np.int64)
    best_t = np.full(len(origins), 1e300)
    for s in range(0, len(origins), chunk):
        o = np.asarray(origins[s:s + chunk], dtype=np.float64)[:, None, :]
        d = np.asarray(directions[s:s + chunk], dtype=np.float64)[:, None, :]
        p = np.cross(d, e2[None])
        det = (e1[None] * p).sum(-1)
        ok = np.abs(det) >= 1e-12
        inv = np.where(ok, 1.0 / np.where(ok, det, 1.0), 0.0)
        t = o - v0[None]
        u = (t * p).sum(-1) * inv
        ok &= (u >= 0.0) & (u <= 1.0)
        q = np.cross(t, e1[None])
        w = (d * q).sum(-1) * inv
        ok &= (w >= 0.0) & (u + w <= 1.0)
        tt = (e2[None] * q).sum(-1) * inv
        ok &= tt > 1e-9
        tt = np.where(ok, tt, 1e300)
        idx = tt.argmin(1)                      # first minimum: ties go to the lower triangle index
        tmin = tt[np.arange(len(idx)), idx]
        hit = tmin < 1e300
        best_f[s:s + chunk] = np.where(hit, idx, -1)
        best_t[s:s + chunk] = tmin
    return best_f, best_t


def render_model(vertices, faces, sgrid):
    """dataset.py:53-95: (3, points) image of distance, n . g and |n ^ g|; face normals from the winding."""
    v = np.asarray(vertices, dtype=np.float64)
    f = np.asarray(faces, dtype=np.int64)
    sgrid = np.asarray(sgrid, dtype=np.float64)
    idx, t = first_hits(v, f, sgrid, -sgrid)
    hit = idx >= 0
    g = sgrid / np.linalg.norm(sgrid, axis=1, keepdims=True)
    loc = sgrid[hit] + t[hit, None] * (-sgrid[hit])
    dist = np.linalg.norm(sgrid[hit] - loc, axis=-1)
    n = np.cross(v[f[:, 1]] - v[f[:, 0]], v[f[:, 2]] - v[f[:, 0]])[idx[hit]]
    n = n / np.linalg.norm(n, axis=1, keepdims=True)
    gh = g[hit]
    dist_im = np.ones(len(sgrid))
    dist_im[hit] = dist
    ndot = np.zeros(len(sgrid))
    ndot[hit] = np.einsum("ij,ij->i", n, gh)
    wedge = np.zeros(len(sgrid))
    nx, ny, nz = n[:, 0], n[:, 1], n[:, 2]
    gx, gy, gz = gh[:, 0], gh[:, 1], gh[:, 2]
    wedge[hit] = np.sqrt((nx * gy - ny * gx) ** 2 + (nx * gz - nz * gx) ** 2 + (ny * gz - nz * gy) ** 2)
    return np.stack((dist_im, ndot, wedge), axis=0)


NORMALISATION = [(0.75, 0.26), (0.59, 0.50), (0.54, 0.29), (0.52, 0.19), (0.80, 0.18), (0.51, 0.25)]   # dataset.py:167-178


def convex_hull_mesh(vertices):
    """Vertices and outward-wound faces of the convex hull (the reference uses trimesh's `mesh.convex_hull`)."""
    from scipy.spatial import ConvexHull
    v = np.asarray(vertices, dtype=np.float64)
    hull = ConvexHull(v)
    faces = hull.simplices.copy()
    n = np.cross(v[faces[:, 1]] - v[faces[:, 0]], v[faces[:, 2]] - v[faces[:, 0]])
    flip = (n * hull.equations[:, :3]).sum(1) < 0
    faces[flip] = faces[flip][:, ::-1]
    return v, faces


def project_on_sphere(vertices, faces, bandwidth, grid_dtype=np.float32):
    """dataset.py:146-182: six channels (mesh and its convex hull), normalised, shape (6, 2b, 2b).  The grid is rounded to
    `grid_dtype` first (the CUDA path reads it as float32): rays that graze a shared edge pick one of two triangles, and
    which one depends on the last bits of the ray."""
    sgrid = make_sgrid(bandwidth).astype(grid_dtype)
    im = render_model(vertices, faces, sgrid)
    hv, hf = convex_hull_mesh(vertices)
    im = np.concatenate([im, render_model(hv, hf, sgrid)], axis=0)
    for c, (mu, sd) in enumerate(NORMALISATION):
        im[c] = (im[c] - mu) / sd
    return im.reshape(6, 2 * bandwidth, 2 * bandwidth).astype(np.float32)
