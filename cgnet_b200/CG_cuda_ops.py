"""The reference extension's six functions, by their own names and argument lists, on top of libcgnet_b200.so.

The reference's Python layer (``CGNet/CG_layers.py:36,65,140,185,199``) imports a compiled module ``CG_cuda_ops``
(``CGNet/cudaCG/cudaCG_all.cpp:207-215``) and hands it tensors it allocated itself together with seven int32 index
tensors.  This module is that interface on the B200 library, so the reference's unmodified ``CG_layers.py`` runs on
these kernels once this module is importable under that name::

    import sys, cgnet_b200.CG_cuda_ops as ops
    sys.modules["CG_cuda_ops"] = ops

    sparse_precomputeCG(CG, L, llls, CG_offsets)                                         cudaCG_all.cpp:112-121
    sparse_forward(F, FF_out, L, B, t_F, cumu_tm_F, t_FF, cumu_tm_FF, llls, l_l1_to_lllidx, t_offsets, CG, CG_offsets)   :39-71
    sparse_backward(F, gF_out, gFF, L, B, t_F, cumu_tm_F, t_FF, cumu_tm_FF, llls, t_offsets, CG, CG_offsets)            :73-108
    sparse_maxL()                                                                        :124-126
    FN_WMM_forward(FF, O_out, W, L, B, size_FN, size_WMM, t_FF, cumu_tm_FF, cumu_tm_O, cumu_tt_W, stds, cnt, eps, flags)  :137-165
    FN_WMM_backward(gO, gFF_out, gW_out, FF, W, L, B, size_FF, size_W, t_FF, cumu_tm_FF, t_O, cumu_tm_O, cumu_tt_W,
                    stds, cnt, eps, flags)                                               :172-205

Every function returns 0 and writes into the caller's output tensors, as the reference's do.  Differences a caller can
observe: the work is enqueued on torch's current stream without a device synchronisation (the reference launches on
the legacy default stream and synchronises after every kernel); outputs are overwritten rather than accumulated into
(the reference's callers always pass zero-filled outputs); the weight gradient is summed in a fixed order; wrong
devices, dtypes or lengths raise ``RuntimeError`` before anything is launched (the reference checks only "CUDA and
contiguous").  The index tensors are read once: their contents select a cached plan (the library's resident form of
the same tables), later calls with the same tensor objects find it without touching the device.
"""
import weakref

import torch

from . import _lib
from .cg_layers import _expect, _ptr, _stream_ptr, get_plan

__all__ = ["sparse_precomputeCG", "sparse_forward", "sparse_backward", "sparse_maxL", "FN_WMM_forward", "FN_WMM_backward"]

# (id of the identifying index tensors) -> (weak references to them, their versions, plan): the fast path of a call
_by_identity = {}


def _host(t):
    return [int(v) for v in t.detach().cpu().reshape(-1).tolist()]


def _lookup(tensors, build):
    key = tuple(id(t) for t in tensors)
    hit = _by_identity.get(key)
    if hit is not None:
        refs, versions, plan = hit
        if all(r() is t for r, t in zip(refs, tensors)) and versions == tuple(t._version for t in tensors):
            return plan
    plan = build()
    if len(_by_identity) > 256:
        _by_identity.clear()
    _by_identity[key] = (tuple(weakref.ref(t) for t in tensors), tuple(t._version for t in tensors), plan)
    return plan


def _product_plan(L, t_F, llls, device):
    """Plan of a product, selected by the contents of the channel counts and the triple codes."""
    return _lookup((t_F, llls), lambda: get_plan(int(L), _host(t_F)[: L + 1], None, _host(llls), device))


def _mixing_plan(L, t_FF, cumu_tm_O, device):
    """Plan of norm + mixing.  The mixing never looks at the pairs, only at the channel counts: one pseudo-triple
    (l, l, l) per degree in channel-wise mode with tau_in = t_FF reproduces exactly those counts."""
    def build():
        tff = _host(t_FF)[: L + 1]
        cum = _host(cumu_tm_O)
        t_O = [(cum[l + 1] - cum[l]) // (2 * l + 1) for l in range(L + 1)]
        L1 = L + 1
        codes = [(l * L1 + l) * L1 + l for l in range(L1) if tff[l] > 0]
        plan = get_plan(int(L), tff, t_O, codes, device, depthwise=True)
        if plan.t_ff() != tff:
            raise RuntimeError("internal: mixing plan disagrees with t_FF")
        return plan
    return _lookup((t_FF, cumu_tm_O), build)


def _int_tensor(t, name):
    if not isinstance(t, torch.Tensor) or t.dtype != torch.int32:
        raise RuntimeError(f"{name} must be an int32 tensor")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")


def sparse_maxL():
    return int(_lib.load().cgb200_max_lmax())


def sparse_precomputeCG(CG_tensor, L, llls, CG_offsets):
    if not CG_tensor.is_cuda or CG_tensor.dtype != torch.float32 or not CG_tensor.is_contiguous():
        raise RuntimeError("CG_tensor must be a contiguous float32 CUDA tensor")
    _int_tensor(llls, "llls")
    codes = _host(llls)
    offs = _host(CG_offsets)
    if len(offs) != len(codes) + 1 or offs[-1] != CG_tensor.numel():
        raise RuntimeError("CG_offsets does not match llls and the length of CG_tensor")
    dev = CG_tensor.device
    with torch.cuda.device(dev):
        _lib.check(_lib.load().cgb200_cg_table_build(_ptr(CG_tensor), CG_tensor.numel(), int(L), _lib.i32(codes), len(codes),
                                                     _stream_ptr(dev)), "cgb200_cg_table_build")
    return 0


def sparse_forward(input, output, L, B, t_F, cumu_tm_F, t_FF, cumu_tm_FF, llls, ll1_to_lllidx, t_offsets, CG, CG_offsets):
    for t, n in ((t_F, "t_F"), (llls, "llls")):
        _int_tensor(t, n)
    plan = _product_plan(L, t_F, llls, input.device)
    plan.check_batch(int(B), input=(input, plan.n_F), output=(output, plan.n_FF))
    with torch.cuda.device(plan.device):
        _lib.check(_lib.load().cgb200_cg_product_fwd(plan.handle, _ptr(input), _ptr(output), int(B), _stream_ptr(plan.device)),
                   "cgb200_cg_product_fwd")
    return 0


def sparse_backward(input, grad_in, grad_out, L, B, t_F, cumu_tm_F, t_FF, cumu_tm_FF, llls, t_offsets, CG, CG_offsets):
    for t, n in ((t_F, "t_F"), (llls, "llls")):
        _int_tensor(t, n)
    plan = _product_plan(L, t_F, llls, input.device)
    plan.check_batch(int(B), input=(input, plan.n_F), grad_in=(grad_in, plan.n_F), grad_out=(grad_out, plan.n_FF))
    with torch.cuda.device(plan.device):
        _lib.check(_lib.load().cgb200_cg_product_bwd(plan.handle, _ptr(input), _ptr(grad_out), _ptr(grad_in), int(B),
                                                     _stream_ptr(plan.device)), "cgb200_cg_product_bwd")
    return 0


def _stds_arg(plan, stds, flags):
    if not (flags & _lib.FN_PRESENT):
        return None   # the reference's callers pass a placeholder tensor in this case; it is never read
    _expect(stds, "FN_stds_tensor", (plan.sum_tff,), plan.device)
    return stds


def FN_WMM_forward(FF_tensor, output_tensor, W_tensor, L, B, size_FN, size_WMM, t_FF, cumu_tm_FF, cumu_tm_O, cumu_tt_W,
                   FN_stds_tensor, FN_cnt, FN_eps, FN_flags):
    for t, n in ((t_FF, "t_FF"), (cumu_tm_O, "cumu_tm_O")):
        _int_tensor(t, n)
    plan = _mixing_plan(L, t_FF, cumu_tm_O, FF_tensor.device)
    flags = int(FN_flags) & (_lib.FN_PRESENT | _lib.FN_UPDATE)
    if int(size_FN) != plan.sum_tff or int(size_WMM) != plan.n_O:
        raise RuntimeError("size_FN / size_WMM do not match the index tensors")
    plan.check_batch(int(B), FF_tensor=(FF_tensor, plan.n_FF), output_tensor=(output_tensor, plan.n_O))
    _expect(W_tensor, "W_tensor", (plan.w_len, 2), plan.device)
    stds = _stds_arg(plan, FN_stds_tensor, flags)
    with torch.cuda.device(plan.device):
        _lib.check(_lib.load().cgb200_fn_wmm_fwd(plan.handle, _ptr(FF_tensor), _ptr(W_tensor), _ptr(stds), float(FN_cnt),
                                                 float(FN_eps), flags, _ptr(output_tensor), int(B), _stream_ptr(plan.device)),
                   "cgb200_fn_wmm_fwd")
    return 0


def FN_WMM_backward(grad_out_tensor, grad_FF_tensor, grad_W_tensor, FF_tensor, W_tensor, L, B, size_FF, size_W, t_FF, cumu_tm_FF,
                    t_O, cumu_tm_O, cumu_tt_W, FN_stds_tensor, FN_cnt, FN_eps, FN_flags):
    for t, n in ((t_FF, "t_FF"), (cumu_tm_O, "cumu_tm_O")):
        _int_tensor(t, n)
    plan = _mixing_plan(L, t_FF, cumu_tm_O, FF_tensor.device)
    flags = int(FN_flags) & _lib.FN_PRESENT
    if int(size_FF) != plan.n_FF or int(size_W) != plan.w_len:
        raise RuntimeError("size_FF / size_W do not match the index tensors")
    plan.check_batch(int(B), FF_tensor=(FF_tensor, plan.n_FF), grad_FF_tensor=(grad_FF_tensor, plan.n_FF),
                     grad_out_tensor=(grad_out_tensor, plan.n_O))
    _expect(W_tensor, "W_tensor", (plan.w_len, 2), plan.device)
    _expect(grad_W_tensor, "grad_W_tensor", (plan.w_len, 2), plan.device)
    stds = _stds_arg(plan, FN_stds_tensor, flags)
    with torch.cuda.device(plan.device):
        _lib.check(_lib.load().cgb200_fn_wmm_bwd(plan.handle, _ptr(grad_out_tensor), _ptr(FF_tensor), _ptr(W_tensor), _ptr(stds),
                                                 float(FN_eps), flags, _ptr(grad_FF_tensor), _ptr(grad_W_tensor), int(B),
                                                 _stream_ptr(plan.device)), "cgb200_fn_wmm_bwd")
    return 0

