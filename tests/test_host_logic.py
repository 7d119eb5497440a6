"""CPU-side tests: the host index layer against the reference fixtures, the C ABI's symbol table, loud failure without a
GPU, and the algorithmic work counts the benchmark reports."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

INDEX_CASES = [("default", 2), ("default", 4), ("default", 5), ("default", 10), ("default", 14),
               ("mst", 2), ("mst", 4), ("mst", 6), ("mst", 10), ("mst", 20), ("debug", 3), ("debug", 5)]


def _ltuples(cgu, mode, L):
    S = cgu.SparseLtuples
    return {"default": S.compute_default_ltuples, "mst": S.compute_mst_ltuples, "debug": S.compute_debug_ltuples}[mode](L)


@pytest.mark.parametrize("mode,L", INDEX_CASES)
def test_host_index_layer_matches_reference(golden_index, mode, L):
    from cgnet_b200 import cgutils as cgu
    g = golden_index
    lt = _ltuples(cgu, mode, L)
    if mode == "mst":
        raw = np.array([(l, a, b) for l in range(L + 1) for a, b in lt[l]], dtype=np.int32)
        np.testing.assert_array_equal(raw, g[f"{mode}_{L}_rawpairs"])
    llls, table = cgu.SparseLtuples.sparse_rep_ltuples_sorted(lt)
    np.testing.assert_array_equal(llls, g[f"{mode}_{L}_llls"])
    np.testing.assert_array_equal(table, g[f"{mode}_{L}_l_l1_offsets"])
    np.testing.assert_array_equal(cgu.SparseLtuples.cal_CG_offsets(L, llls), g[f"{mode}_{L}_cg_offsets"])
    assert cgu.SparseLtuples.get_CG_length(L, llls) == g[f"{mode}_{L}_cg_offsets"][-1]
    for tag in ("ones", "ramp"):
        taus = g[f"{mode}_{L}_{tag}_taus"]
        t_ff, offs = cgu.SparseLtuples.cal_new_tau_and_offsets(L, taus, llls)
        np.testing.assert_array_equal(t_ff, g[f"{mode}_{L}_{tag}_tFF"])
        np.testing.assert_array_equal(offs, g[f"{mode}_{L}_{tag}_toffsets"])
    assert cgu.SparseLtuples.get_iter(L, llls)[0][0] == 0


def test_reshape_and_products():
    from cgnet_b200 import cgutils as cgu
    taus = [2, 1, 3]
    x = torch.arange(2 * (2 + 3 + 15) * 2, dtype=torch.float32).reshape(2, 20, 2)
    parts = cgu.reshape_out(x, taus)
    assert [tuple(p.shape) for p in parts] == [(2, 2, 1, 2), (2, 1, 3, 2), (2, 3, 5, 2)]
    assert torch.equal(torch.cat([p.reshape(2, -1, 2) for p in parts], 1), x)
    assert cgu.calc_prod_taus(2, [2, 1, 1]) == [6, 5, 5]
    w = torch.randn(3, 2, 4, 2)
    f = torch.randn(3, 4, 5, 2)
    want = torch.view_as_real(torch.matmul(torch.view_as_complex(w), torch.view_as_complex(f)))
    assert torch.allclose(cgu.Complex_bmm(w, f), want)
    assert cgu.cumulative_tm([2, 1, 3]).tolist() == [0, 2, 5, 20]


def test_library_exports_every_declared_symbol():
    from cgnet_b200 import _lib
    header = open(os.path.join(ROOT, "include", "cgnet_b200.h")).read()
    header = re.sub(r"/\*.*?\*/", "", header, flags=re.S)
    declared = set(re.findall(r"\b(cgb200_[a-z_0-9]+)\s*\(", header))
    assert len(declared) >= 20
    lib = ctypes.CDLL(_lib.LIB_PATH)
    for name in sorted(declared):
        assert hasattr(lib, name), f"{name} is declared in include/cgnet_b200.h but not exported"
    assert declared == set(_lib.SIGNATURES), "ctypes signature table and header disagree"
    loaded = _lib.load()
    assert loaded.cgb200_version() >= 100 and loaded.cgb200_max_lmax() == 511
    assert loaded.cgb200_kernel_count() >= 18
    assert loaded.cgb200_kernel_name(9) == b"fused_fwd"


def test_table_length_and_argument_checks_need_no_gpu():
    from cgnet_b200 import _lib
    from cgnet_b200 import cgutils as cgu
    lib = _lib.load()
    llls, _ = cgu.SparseLtuples.sparse_rep_ltuples_sorted(cgu.SparseLtuples.compute_default_ltuples(10))
    assert lib.cgb200_cg_table_length(10, _lib.i32(llls), len(llls)) == 49535
    # l2 > l1 is refused before any CUDA call
    bad = [(0 * 3 + 1) * 3 + 2]
    assert lib.cgb200_cg_table_length(2, _lib.i32(bad), 1) == -1
    assert b"l2 <= l1" in lib.cgb200_last_error()
    h = _lib.vp()
    assert lib.cgb200_plan_create(h, 600, _lib.i32([1]), None, _lib.i32([0]), 1, 0) == 1   # lmax beyond 511
    assert lib.cgb200_layer_workspace_bytes(None, 4) == -1


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the behaviour of a machine without a GPU")
def test_modules_fail_loudly_without_a_gpu():
    from cgnet_b200 import CGBN_cuda
    with pytest.raises(RuntimeError):
        CGBN_cuda(2, [2, 2, 2], [2, 2, 2], device="cuda")


def test_argument_checks_raise_before_any_launch():
    """Wrong lengths, dtypes, devices and layouts must be Python errors, never pointers handed to a kernel."""
    from cgnet_b200 import _lib
    from cgnet_b200.cg_layers import PlanShapes
    dev = torch.device("cpu")   # the checks compare devices, they do not need a GPU to be exercised
    shapes = PlanShapes(dev, n_F=20, n_FF=46, n_O=12, w_len=30, sum_tff=16)
    F = torch.zeros(3, 20, 2)
    W = torch.zeros(30, 2)
    stds = torch.ones(16)
    shapes.check_batch(3, F=(F, 20))
    shapes.check_weights(W, stds, _lib.FN_PRESENT)
    shapes.check_weights(W, None, 0)
    with pytest.raises(RuntimeError, match="shape"):
        shapes.check_batch(3, F=(torch.zeros(3, 19, 2), 20))            # activation of the wrong length
    with pytest.raises(RuntimeError, match="shape"):
        shapes.check_batch(3, F=(F, 20), gO=(torch.zeros(2, 12, 2), 12))  # cotangent with another batch size
    with pytest.raises(RuntimeError, match="shape"):
        shapes.check_weights(torch.zeros(29, 2), stds, _lib.FN_PRESENT)
    with pytest.raises(RuntimeError, match="shape"):
        shapes.check_weights(W, torch.ones(15), _lib.FN_PRESENT)
    with pytest.raises(RuntimeError, match="float32"):
        shapes.check_weights(W, stds.half(), _lib.FN_PRESENT)           # what model.half() would do to the statistics
    with pytest.raises(RuntimeError, match="float32"):
        shapes.check_batch(3, F=(F.double(), 20))
    with pytest.raises(RuntimeError, match="None"):
        shapes.check_weights(W, None, _lib.FN_PRESENT)
    with pytest.raises(RuntimeError, match="contiguous"):
        shapes.check_batch(3, F=(torch.zeros(3, 2, 20).transpose(1, 2), 20))
    with pytest.raises(RuntimeError, match="lives on"):
        PlanShapes(torch.device("meta"), 20, 46, 12, 30, 16).check_batch(3, F=(F, 20))   # tensor on another device than the plan


def test_plan_options_are_checked_without_a_gpu():
    from cgnet_b200 import _lib
    lib = _lib.load()
    assert lib.cgb200_plan_set_option(None, 0, 1) == 1
    v = ctypes.c_int32(0)
    assert lib.cgb200_plan_get_option(None, 0, v) == 1
    assert lib.cgb200_layer_fwd_workspace_bytes(None, 4) == -1


def test_benchmark_work_counts():
    import bench
    w = bench.layer_work(10, [5] * 11, [5] * 11)
    assert w["n_FF"] == 118525 and w["n_F"] == 605 and w["w_len"] == 47625 and w["cg_len"] == 49535
    assert abs(w["cg_flops"] / 8.26e6 - 1) < 0.01 and abs(w["mix_flops"] / 4.74e6 - 1) < 0.01
    w0 = bench.layer_work(10, [1] * 11, [5] * 11)
    assert w0["n_FF"] == 4741 and w0["w_len"] == 1905
    w1 = bench.layer_work(5, [8] * 6, [8] * 6)
    assert w1["n_FF"] == 29248 and w1["w_len"] == 35328
