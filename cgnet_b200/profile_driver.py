"""One launch of every kernel family of libcgnet_b200.so, for a profiler to capture.

    python -m cgnet_b200.profile_driver                      # runs by itself: every call returns, statuses are checked
    ncu --set full --clock-control none -k regex:'cg_fwd|cg_bwd|fn_stats|wmm_|prep_kernel|tc_pack|fused_|gff_|sh_pack|sh_project|reduce_kernel|raycast' \\
        -c 48 -o all_kernels python -m cgnet_b200.profile_driver

Cases (seeded random inputs; the two-pass case is sized so that the mid activation, 190 MB, exceeds the 126 MB L2):
  two-pass product / statistics / mixing and their gradients   lmax 10, 5 channels, batch 200
  fused layer forward (training statistics) + backward         the same layer (CUDA-core kernels)
  fused layer forward + backward                               lmax 10, 16 channels, batch 128 (tensor-core forward, weight gradient
                                                               and mid-gradient GEMM)
  spherical-harmonic projection                                4096 points, lmax 14, 768 functions
  mesh -> sphere ray casting                                   a 5120-triangle sphere mesh, 64 x 64 grid
"""
import numpy as np
import torch

from . import CGutils, _lib, get_plan
from .s2_sph import SHProjector
from .shrec_project import make_sgrid, render_model


def _layer_case(lmax, tau, batch, dev, rng):
    llls = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(CGutils.SparseLtuples.compute_default_ltuples(lmax))[0]
    plan = get_plan(lmax, [tau] * (lmax + 1), [tau] * (lmax + 1), llls, dev)
    F = torch.tensor(rng.randn(batch, plan.n_F, 2).astype(np.float32), device=dev)
    W = torch.tensor((0.05 * rng.rand(plan.w_len, 2)).astype(np.float32), device=dev)
    stds = torch.tensor((0.25 + rng.rand(plan.sum_tff)).astype(np.float32), device=dev)
    gO = torch.tensor(rng.randn(batch, plan.n_O, 2).astype(np.float32), device=dev)
    return plan, F, W, stds, gO


def _sphere_mesh(subdiv):
    t = (1.0 + 5 ** 0.5) / 2.0
    v = [np.array(x, dtype=np.float64) for x in ((-1, t, 0), (1, t, 0), (-1, -t, 0), (1, -t, 0), (0, -1, t), (0, 1, t), (0, -1, -t),
                                                 (0, 1, -t), (t, 0, -1), (t, 0, 1), (-t, 0, -1), (-t, 0, 1))]
    v = [x / np.linalg.norm(x) for x in v]
    f = [(0, 11, 5), (0, 5, 1), (0, 1, 7), (0, 7, 10), (0, 10, 11), (1, 5, 9), (5, 11, 4), (11, 10, 2), (10, 7, 6), (7, 1, 8),
         (3, 9, 4), (3, 4, 2), (3, 2, 6), (3, 6, 8), (3, 8, 9), (4, 9, 5), (2, 4, 11), (6, 2, 10), (8, 6, 7), (9, 8, 1)]
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
    return (0.99 * np.array(v)).astype(np.float32), np.array(f, dtype=np.int32)


def main():
    dev = torch.device("cuda", 0)
    rng = np.random.RandomState(0)
    flags_train = _lib.FN_PRESENT | _lib.FN_UPDATE
    plan, F, W, stds, gO = _layer_case(10, 5, 200, dev, rng)
    FF = plan.cg_product_fwd(F)
    plan.fn_wmm_fwd(FF, W, stds, 2.0, 1e-5, flags_train)
    gFF, _ = plan.fn_wmm_bwd(gO, FF, W, stds, 1e-5, _lib.FN_PRESENT)
    plan.cg_product_bwd(F, gFF)
    plan.layer_fwd(F, W, stds, 2.0, 1e-5, flags_train)
    plan.layer_bwd(F, W, stds, 1e-5, _lib.FN_PRESENT, gO)
    p16, F16, W16, s16, g16 = _layer_case(10, 16, 128, dev, rng)
    p16.layer_fwd(F16, W16, s16, 2.0, 1e-5, flags_train)
    p16.layer_bwd(F16, W16, s16, 1e-5, _lib.FN_PRESENT, g16)
    P = 4096
    proj = SHProjector(15, rng.uniform(0, np.pi, P), rng.uniform(0, 2 * np.pi, P), conjugate=False, device=dev)
    proj.project(torch.tensor(rng.randn(768, P).astype(np.float32), device=dev))
    v, f = _sphere_mesh(4)
    render_model(v, f, make_sgrid(32), dev)
    torch.cuda.synchronize()
    plan.check_status()
    p16.check_status()
    proj.check_status()
    print("profile driver: every kernel family launched once")


if __name__ == "__main__":
    main()
