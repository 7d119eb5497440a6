"""The CPU oracle against the fixtures produced by the reference's own CPU code (tests/golden/make_golden.py), against
sympy's exact Clebsch-Gordan coefficients, and against algebraic identities of the coefficients."""
import numpy as np
import pytest
import torch

import cg_oracle as o

INDEX_CASES = [("default", 2), ("default", 4), ("default", 5), ("default", 10), ("default", 14),
               ("mst", 2), ("mst", 4), ("mst", 6), ("mst", 10), ("mst", 20), ("debug", 3), ("debug", 5)]
LAYER_CASES = ["t21_mst", "t21_default", "t32111_default", "t32111_mst", "t211_default", "t2222_debug",
               "L5t4_default", "L6ragged_mst"]


def ltuples_for(mode, L):
    return {"default": o.default_ltuples, "mst": o.mst_ltuples, "debug": o.debug_ltuples}[mode](L)


def rel_fro(a, b):
    a = np.asarray(a, dtype=np.float64)
    b = np.asarray(b, dtype=np.float64)
    d = np.linalg.norm(b)
    return np.linalg.norm(a - b) / d if d > 0 else np.linalg.norm(a)


@pytest.mark.parametrize("mode,L", INDEX_CASES)
def test_index_layer_matches_reference(golden_index, mode, L):
    g = golden_index
    lt = ltuples_for(mode, L)
    if mode == "mst":
        raw = np.array([(l, a, b) for l in range(L + 1) for a, b in lt[l]], dtype=np.int32)
        np.testing.assert_array_equal(raw, g[f"{mode}_{L}_rawpairs"])
    llls, table = o.encode_sorted(lt)
    np.testing.assert_array_equal(llls, g[f"{mode}_{L}_llls"])
    np.testing.assert_array_equal(table, g[f"{mode}_{L}_l_l1_offsets"])
    np.testing.assert_array_equal(o.cg_offsets(L, llls), g[f"{mode}_{L}_cg_offsets"])
    for tag in ("ones", "ramp"):
        taus = g[f"{mode}_{L}_{tag}_taus"]
        t_ff, offs = o.tau_ff_and_offsets(L, taus, llls)
        np.testing.assert_array_equal(t_ff, g[f"{mode}_{L}_{tag}_tFF"])
        np.testing.assert_array_equal(offs, g[f"{mode}_{L}_{tag}_toffsets"])


def test_index_known_answers():
    # triples of lmax=2 in canonical order, and the per-degree channel counts for taus=[2,1,1]
    llls, _ = o.encode_sorted(o.default_ltuples(2))
    assert o.decode_triples(2, llls) == [(0, 0, 0), (0, 1, 1), (0, 2, 2), (1, 1, 0), (1, 1, 1), (1, 2, 1), (1, 2, 2),
                                         (2, 1, 1), (2, 2, 0), (2, 2, 1), (2, 2, 2)]
    t_ff, _ = o.tau_ff_and_offsets(2, [2, 1, 1], llls)
    assert t_ff.tolist() == [6, 5, 5]
    for L, n in ((5, 69), (10, 381), (14, 932), (20, 2486), (30, 7816)):
        assert len(o.encode_sorted(o.default_ltuples(L))[0]) == n
    assert len(o.encode_sorted(o.mst_ltuples(20))[0]) == 731
    # MNIST example of the reference (lmax 10, taus ceil(12/sqrt(2l+1))): weight sizes quoted in MNIST/example.sh:12
    taus = [12, 7, 6, 5, 4, 4, 4, 4, 3, 3, 3]
    llls, _ = o.encode_sorted(o.default_ltuples(10))
    t0, _ = o.tau_ff_and_offsets(10, [1] * 11, llls)
    t1, _ = o.tau_ff_and_offsets(10, taus, llls)
    assert int((t0 * np.array(taus)).sum()) == 1643 and int((t1 * np.array(taus)).sum()) == 31023


def test_cg_dense_matches_reference_module(golden_cg):
    g = golden_cg
    n = 0
    for key in g.files:
        if key.startswith("dense_L4_"):
            l1, l2, l = (int(x) for x in key.split("_")[2:])
            np.testing.assert_allclose(o.cg_dense(l1, l2, l), g[key], atol=1e-13, rtol=0)
            n += 1
    assert n == 65
    for L in (10, 20):
        keys = g[f"dense_L{L}_keys"]
        for i in range(0, len(keys), 7 if L == 20 else 1):
            idx = int(keys[i])
            l, l2, l1 = idx % (L + 1), (idx // (L + 1)) % (L + 1), idx // (L + 1) ** 2
            M = o.cg_dense(l1, l2, l)
            w = np.cos(np.arange(M.size).reshape(M.shape) * 0.37)
            assert abs(M.sum() - g[f"dense_L{L}_sum"][i]) < 1e-9
            assert abs(np.abs(M).sum() - g[f"dense_L{L}_abs"][i]) < 1e-9
            assert abs((M * w).sum() - g[f"dense_L{L}_wsum"][i]) < 1e-9


def test_cg_band_table_matches_reference_builder(golden_cg):
    for L in (3, 6):
        llls, _ = o.encode_sorted(o.default_ltuples(L))
        band, offs = o.cg_band_table(L, llls)
        assert offs[-1] == golden_cg[f"band_default_{L}"].shape[0]
        np.testing.assert_allclose(band, golden_cg[f"band_default_{L}"], atol=1e-7, rtol=0)


def test_cg_against_sympy_exact():
    from sympy import S
    from sympy.physics.quantum.cg import CG
    worst = 0.0
    for l1 in range(4):
        for l2 in range(l1 + 1):
            for l in range(l1 - l2, l1 + l2 + 1):
                for m1 in range(-l1, l1 + 1):
                    for m2 in range(-l2, l2 + 1):
                        if abs(m1 + m2) > l:
                            continue
                        exact = float(CG(S(l1), S(m1), S(l2), S(m2), S(l), S(m1 + m2)).doit())
                        worst = max(worst, abs(exact - o.cg_coeff(l1, l2, l, m1, m2)))
    assert worst < 1e-13
    # the two values a maintainer can check by hand
    assert abs(o.cg_coeff(1, 1, 0, 1, -1) - 1 / np.sqrt(3)) < 1e-14
    assert abs(o.cg_coeff(1, 1, 1, -1, 0) + 1 / np.sqrt(2)) < 1e-14


@pytest.mark.parametrize("L", [6, 16, 30])
def test_cg_rows_orthonormal(L):
    # sum over (m1,m2) of C[m,(m1,m2)] C[m',(m1,m2)] = delta_mm' for every admissible triple
    worst = 0.0
    rng = np.random.RandomState(L)
    triples = [(l1, l2, l) for l1 in range(L + 1) for l2 in range(l1 + 1) for l in range(l1 - l2, min(l1 + l2, L) + 1)]
    if len(triples) > 300:
        keep = rng.choice(len(triples), 300, replace=False)
        triples = [triples[i] for i in keep] + [(L, L, L), (L, L, 0), (L, 0, L)]
    for l1, l2, l in triples:
        M = o.cg_dense(l1, l2, l)
        worst = max(worst, np.abs(M @ M.T - np.eye(2 * l + 1)).max())
    assert worst < 5e-9


@pytest.mark.parametrize("name", LAYER_CASES)
def test_layer_matches_reference_twin(golden_layers, name):
    g = {k.split("/", 1)[1]: golden_layers[k] for k in golden_layers.files if k.startswith(name + "/")}
    taus, tau_out, llls = g["taus"].tolist(), g["tau_out"].tolist(), g["llls"].tolist()
    L = len(taus) - 1
    tol = 2e-6  # fp32 twin vs fp32 oracle: same arithmetic up to summation order

    def fresh():
        F = torch.tensor(g["F"], requires_grad=True)
        W = torch.tensor(g["W"], requires_grad=True)
        return F, W, o.split_fragments(F, taus)

    # CG product and its input gradient
    F, W, frags = fresh()
    ff = o.join_fragments(o.cg_product(frags, taus, L, llls))
    if "FF" in g:
        assert rel_fro(ff.detach().numpy(), g["FF"]) < tol
        g_ff = torch.tensor(g["gFF"])
    else:
        g_ff = torch.tensor(np.random.RandomState(1234).randn(*ff.shape), dtype=torch.float)
        t_ff, _ = o.tau_ff_and_offsets(L, taus, llls)
        norms = [float(f.norm()) for f in o.split_fragments(ff.detach(), t_ff)]
        np.testing.assert_allclose(norms, g["FF_fragnorm"], rtol=1e-5)
        assert abs(float((ff.detach().double() * g_ff.double()).sum()) - float(g["FF_proj"])) < 1e-4 * abs(float(g["FF_proj"])) + 1e-3
    (ff * g_ff).sum().backward()
    assert rel_fro(F.grad.numpy(), g["cg_gF"]) < tol

    g_o = torch.tensor(g["gO"])
    for key, stds, training in (("nobn", None, False), ("bneval", g["stds"], False), ("harness_bntrain", g["stds"], True)):
        F, W, frags = fresh()
        out, new_stds = o.cgbn_layer(frags, taus, tau_out, L, llls, W, stds=stds, eps=1e-5, cnt=1.0, training=training)
        O = o.join_fragments(out)
        assert rel_fro(O.detach().numpy(), g[f"{key}_O"]) < 5e-6, key
        (O * g_o).sum().backward()
        assert rel_fro(F.grad.numpy(), g[f"{key}_gF"]) < 5e-6, key
        assert rel_fro(W.grad.numpy(), g[f"{key}_gW"]) < 5e-6, key
        if training:
            # the twin takes np.std of an fp32 array (fp32 accumulation); the oracle and the CUDA reference use double
            np.testing.assert_allclose(new_stds, g["harness_bntrain_stds"], rtol=2e-5, atol=1e-6)


def test_twin_style_forward_equals_oracle(golden_layers):
    name = "t32111_mst"
    g = {k.split("/", 1)[1]: golden_layers[k] for k in golden_layers.files if k.startswith(name + "/")}
    taus, tau_out, llls = g["taus"].tolist(), g["tau_out"].tolist(), g["llls"].tolist()
    F = torch.tensor(g["F"])
    W = torch.tensor(g["W"])
    out = o.twin_forward(o.split_fragments(F, taus), taus, tau_out, len(taus) - 1, llls, W, stds=g["stds"])
    assert rel_fro(o.join_fragments(out).numpy(), g["bneval_O"]) < 5e-6


def test_depthwise_is_the_diagonal_of_the_full_product():
    taus = [3, 3, 3]
    llls, _ = o.encode_sorted(o.default_ltuples(2))
    rng = np.random.RandomState(3)
    frags = [torch.tensor(rng.randn(2, 3, 2 * l + 1, 2), dtype=torch.float64) for l in range(3)]
    full = o.cg_product(frags, taus, 2, llls)
    dw = o.cg_product(frags, taus, 2, llls, depthwise=True)
    for l in range(3):
        n_tr = full[l].shape[1] // 9
        idx = [k * 9 + t * 3 + t for k in range(n_tr) for t in range(3)]
        assert torch.allclose(full[l][:, idx], dw[l])
