"""The mesh -> sphere ray casting of the SHREC17 front end against the CPU restatement of the reference's `render_model`
/ `ProjectOnSphere` on synthetic meshes (the data set itself is not distributed with the reference).  Hit / miss and the
triangle hit must agree exactly (both sides evaluate the same float64 test on the same float32 inputs); the image values
to 1e-5."""
import numpy as np
import pytest
import torch

import raycast_oracle as ro


def icosphere(subdiv, seed=0, bumpy=0.0):
    """Unit icosahedron subdivided `subdiv` times, outward winding, optionally with radial noise (a star-shaped mesh)."""
    t = (1.0 + 5 ** 0.5) / 2.0
    v = [(-1, t, 0), (1, t, 0), (-1, -t, 0), (1, -t, 0), (0, -1, t), (0, 1, t), (0, -1, -t), (0, 1, -t), (t, 0, -1), (t, 0, 1), (-t, 0, -1), (-t, 0, 1)]
    f = [(0, 11, 5), (0, 5, 1), (0, 1, 7), (0, 7, 10), (0, 10, 11), (1, 5, 9), (5, 11, 4), (11, 10, 2), (10, 7, 6), (7, 1, 8),
         (3, 9, 4), (3, 4, 2), (3, 2, 6), (3, 6, 8), (3, 8, 9), (4, 9, 5), (2, 4, 11), (6, 2, 10), (8, 6, 7), (9, 8, 1)]
    v = [np.array(x, dtype=np.float64) / np.linalg.norm(x) for x in v]
    for _ in range(subdiv):
        cache, nf = {}, []

        def mid(a, b):
            key = (min(a, b), max(a, b))
            if key not in cache:
                m = v[a] + v[b]
                v.append(m / np.linalg.norm(m))
                cache[key] = len(v) - 1
            return cache[key]
        for a, b, c in f:
            ab, bc, ca = mid(a, b), mid(b, c), mid(c, a)
            nf += [(a, ab, ca), (b, bc, ab), (c, ca, bc), (ab, bc, ca)]
        f = nf
    v = np.array(v)
    if bumpy:
        v = v * (1.0 + bumpy * np.random.RandomState(seed).rand(len(v), 1))
    v = v * (0.99 / np.linalg.norm(v, axis=1).max())     # the reference scales meshes into the 0.99 ball (dataset.py:136-137)
    return v.astype(np.float32), np.array(f, dtype=np.int32)


def test_oracle_on_a_sphere_mesh():
    """A fine sphere mesh of radius ~0.99: every ray hits, distance ~0.01, normal along the ray."""
    v, f = icosphere(3)
    im = ro.render_model(v, f, ro.make_sgrid(6))
    assert im.shape == (3, 144)
    assert np.all(im[0] < 0.03) and np.all(im[0] > 0.0099)
    assert np.all(im[1] > 0.99) and np.all(im[2] < 0.15)


@pytest.mark.gpu
@pytest.mark.parametrize("subdiv,bumpy,b", [(2, 0.0, 8), (3, 0.4, 16), (1, 0.8, 5)])
def test_render_model_matches_restatement(subdiv, bumpy, b):
    from cgnet_b200.shrec_project import make_sgrid, render_model
    v, f = icosphere(subdiv, seed=b, bumpy=bumpy)
    sgrid = make_sgrid(b, 0.3, 0.7, 1.1)
    np.testing.assert_allclose(sgrid, ro.make_sgrid(b, 0.3, 0.7, 1.1), atol=1e-15)
    got = render_model(v, f, sgrid, torch.device("cuda", 0)).cpu().numpy()
    want = ro.render_model(v, f, sgrid.astype(np.float32))     # the kernel reads the grid as float32
    assert got.shape == want.shape == (3, (2 * b) ** 2)
    assert np.array_equal(got[0] == 1.0, want[0] == 1.0), "hit / miss differs"
    np.testing.assert_allclose(got, want, atol=1e-5, rtol=0)


@pytest.mark.gpu
def test_open_mesh_rays_that_miss_and_empty_mesh():
    from cgnet_b200.shrec_project import make_sgrid, render_model
    dev = torch.device("cuda", 0)
    v, f = icosphere(2)
    f = f[: len(f) // 3]                                   # an open cap: most rays meet nothing
    sgrid = make_sgrid(8)
    got = render_model(v, f, sgrid, dev).cpu().numpy()
    want = ro.render_model(v, f, sgrid.astype(np.float32))
    assert (want[0] == 1.0).sum() > 50
    assert np.array_equal(got[0] == 1.0, want[0] == 1.0)
    np.testing.assert_allclose(got, want, atol=1e-5, rtol=0)
    empty = render_model(np.zeros((0, 3), np.float32), np.zeros((0, 3), np.int32), sgrid, dev).cpu().numpy()
    assert np.all(empty[0] == 1.0) and np.all(empty[1:] == 0.0)


@pytest.mark.gpu
def test_project_on_sphere_six_channels():
    from cgnet_b200.shrec_project import ProjectOnSphere
    v, f = icosphere(2, seed=3, bumpy=0.6)
    got = ProjectOnSphere(8, device=torch.device("cuda", 0))(v, f).cpu().numpy()
    want = ro.project_on_sphere(v, f, 8)
    assert got.shape == (6, 16, 16) and got.dtype == np.float32
    np.testing.assert_allclose(got, want, atol=2e-5, rtol=0)
