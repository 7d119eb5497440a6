"""The Clebsch-Gordan layer modules, API-compatible with the reference's ``CGNet/CG_layers.py``:

    CGBN_cuda            CG product -> fragment norm -> per-degree complex channel mixing   (CG_layers.py:289-318)
    CG_woFilter_cuda     the CG product alone                                               (CG_layers.py:205-286)
    MyBatchNormWeightMM_cuda   fragment norm + mixing on a materialised product             (CG_layers.py:74-132)
    precomputeCG         cached CG band table for a degree cut-off                          (CG_layers.py:153-165)

Constructor arguments, attribute names, parameter names/shapes (``W``, ``bn_stds``, ``bn_eps``) and the
list-or-flat calling convention are the reference's, so a model written against it runs unchanged and its
checkpoints load.  All arithmetic happens in libcgnet_b200.so (hand-written sm_100a kernels behind a C ABI); torch
supplies device memory, the current stream and autograd bookkeeping only.  There is no CPU path: tensors must live on
a CUDA device.

Differences from the reference, all additive:
  * ``CGBN_cuda`` runs the whole layer through fused kernels that never write the quadratic mid activation to memory
    (``fused=False`` selects the two-pass route through ``self.cg`` and ``self.bnWMM``);
  * ``device`` is honoured everywhere (the reference hard-codes ``'cuda'`` in places);
  * ``bn_cnt`` is also kept in a buffer so that it survives ``state_dict`` round trips (reference: a Python float that
    a resume silently resets, ``CG_layers.py:92``); checkpoints without it still load;
  * ``depthwise=True`` (channel-wise product, tau_l1 == tau_l2 required) is an extension with no reference counterpart;
  * ``keep_mid`` (``CGBN_cuda``): wide layers in training keep their workspace, with the mid activation's tiles in it, from
    the forward to the backward (default: while the workspaces kept on the device stay under a quarter of its memory);
  * gradients of ``W`` are summed in a fixed order (the reference accumulates them with ``atomicAdd``).
"""
import functools
import weakref

import numpy as np
import torch
from torch import nn

from . import _lib
from . import cgutils as CGutils

__all__ = ["CGBN_cuda", "CG_woFilter_cuda", "MyBatchNormWeightMM_cuda", "precomputeCG", "Plan", "PlanShapes", "get_plan"]


def _stream_ptr(device):
    return torch.cuda.current_stream(device).cuda_stream


def _ptr(t):
    return None if t is None else t.data_ptr()


_raw_stream = getattr(torch._C, "_cuda_getCurrentRawStream", None)


def _current_stream(index):
    """Handle of PyTorch's current stream on device ``index``.  The raw getter skips building a ``torch.cuda.Stream``
    object, which costs several microseconds on a path that runs twice per layer and step."""
    if _raw_stream is not None:
        return _raw_stream(index)
    return torch.cuda.current_stream(index).cuda_stream


def _check_cuda_f32(t, name):
    if not isinstance(t, torch.Tensor) or not t.is_cuda:
        raise RuntimeError(f"{name} must be a CUDA tensor (cgnet_b200 has no CPU path)")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32, got {t.dtype}")
    return t.contiguous()


def _expect(t, name, shape_tail, device, allow_none=False):
    """Raise unless ``t`` is a contiguous float32 tensor on ``device`` whose trailing dimensions are ``shape_tail``
    (the leading one is the batch).  Runs before any pointer reaches the library: a wrong length or a tensor on
    another GPU would otherwise be an out-of-bounds or peer access inside a kernel."""
    if t is None:
        if allow_none:
            return
        raise RuntimeError(f"{name} is None")
    if not isinstance(t, torch.Tensor):
        raise RuntimeError(f"{name} must be a tensor, got {type(t).__name__}")
    if t.dtype != torch.float32:
        raise RuntimeError(f"{name} must be float32, got {t.dtype}")
    if t.device != device:
        raise RuntimeError(f"{name} lives on {t.device}, the plan on {device}")
    if not t.is_contiguous():
        raise RuntimeError(f"{name} must be contiguous")
    nd, k = t.dim(), len(shape_tail)
    if nd < k or nd > k + 1 or tuple(t.shape[nd - k:]) != tuple(shape_tail):
        raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected (..., {', '.join(str(x) for x in shape_tail)})")


class PlanShapes:
    """The sizes a plan fixes and the argument checks that follow from them (kept apart from the device handle so that
    the checks can be exercised without a GPU)."""

    def __init__(self, device, n_F, n_FF, n_O, w_len, sum_tff):
        self.device = torch.device(device)
        self.n_F, self.n_FF, self.n_O, self.w_len, self.sum_tff = int(n_F), int(n_FF), int(n_O), int(w_len), int(sum_tff)

    def check_weights(self, W, stds, flags):
        _expect(W, "W", (self.w_len, 2), self.device)
        if flags & _lib.FN_PRESENT:
            _expect(stds, "bn_stds", (self.sum_tff,), self.device)

    def check_batch(self, B, **named):
        """named: name=(tensor, per-sample length); all must share the batch size B."""
        for name, (t, n) in named.items():
            _expect(t, name, (n, 2), self.device)
            if t.dim() != 3 or t.shape[0] != B:
                raise RuntimeError(f"{name} has shape {tuple(t.shape)}, expected ({B}, {n}, 2)")


class Plan(PlanShapes):
    """Owner of one ``cgb200_plan`` handle: index tables, CG table and work lists for a fixed
    (lmax, tau_in, tau_out, triple list) on one device."""

    def __init__(self, lmax, taus, tau_out, llls, device, depthwise=False, tile=0):
        lib = _lib.load()
        device = torch.device(device)
        if device.type != "cuda":
            raise RuntimeError("cgnet_b200 plans live on a CUDA device")
        if device.index is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.device = device
        self.lmax = int(lmax)
        if self.lmax > lib.cgb200_max_lmax():
            raise AssertionError(f"Does not support lmax={lmax}")
        handle = _lib.vp()
        a_in = _lib.i32(taus)
        a_out = _lib.i32(tau_out) if tau_out is not None else None
        a_l = _lib.i32(llls)
        flags = (_lib.PLAN_DEPTHWISE if depthwise else 0) | _lib.plan_tile_flag(tile)
        with torch.cuda.device(self.device):
            _lib.check(lib.cgb200_plan_create(handle, self.lmax, a_in, a_out, a_l, len(llls), flags), "cgb200_plan_create")
        self.handle = handle
        self._finalizer = weakref.finalize(self, lib.cgb200_plan_destroy, handle)
        super().__init__(self.device, self.query(_lib.Q_N_F), self.query(_lib.Q_N_FF), self.query(_lib.Q_N_O),
                         self.query(_lib.Q_W_LEN), self.query(_lib.Q_SUM_TFF))
        self.tile = self.query(_lib.Q_TILE)
        self._ws_bytes = {}
        self._option_epoch = 0      # bumped by set_option: whatever was derived from the options is stale then
        self._fn_layer_fwd, self._fn_layer_bwd = lib.cgb200_layer_fwd, lib.cgb200_layer_bwd

    def query(self, what):
        v = _lib.ctypes.c_int64()
        _lib.check(_lib.load().cgb200_plan_query(self.handle, what, v), "cgb200_plan_query")
        return int(v.value)

    def t_ff(self):
        out = (_lib.ctypes.c_int32 * (self.lmax + 1))()
        _lib.check(_lib.load().cgb200_plan_t_ff(self.handle, out), "cgb200_plan_t_ff")
        return list(out)

    def set_option(self, option, value):
        """Select a kernel variant for this plan (``_lib.OPT_*``; ``_lib.AUTO`` restores the library's default)."""
        _lib.check(_lib.load().cgb200_plan_set_option(self.handle, int(option), int(value)), "cgb200_plan_set_option")
        self._ws_bytes.clear()
        self._option_epoch += 1

    def get_option(self, option):
        v = _lib.ctypes.c_int32()
        _lib.check(_lib.load().cgb200_plan_get_option(self.handle, int(option), v), "cgb200_plan_get_option")
        return int(v.value)

    def check_status(self):
        """Raise if a kernel of this plan gave up on a bounded device-side wait since the last check (its outputs were
        then filled with NaN).  Synchronises the device: call it once per epoch or checkpoint, not per step."""
        st = _lib.ctypes.c_int32(-1)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().cgb200_plan_status(self.handle, st), "cgb200_plan_status")
        if st.value != 0:
            raise RuntimeError("a cgnet_b200 tensor-core kernel gave up on a bounded wait; the outputs of that call are NaN")

    # ---- thin wrappers over the C ABI: arguments are checked against the plan's sizes and device before any launch ----
    def cg_product_fwd(self, F):
        B = F.shape[0]
        self.check_batch(B, F=(F, self.n_F))
        FF = torch.empty(B, self.n_FF, 2, device=F.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().cgb200_cg_product_fwd(self.handle, _ptr(F), _ptr(FF), B, _stream_ptr(self.device)),
                       "cgb200_cg_product_fwd")
        return FF

    def cg_product_bwd(self, F, gFF):
        self.check_batch(F.shape[0], F=(F, self.n_F), gFF=(gFF, self.n_FF))
        gF = torch.empty_like(F)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().cgb200_cg_product_bwd(self.handle, _ptr(F), _ptr(gFF), _ptr(gF), F.shape[0],
                                                         _stream_ptr(self.device)), "cgb200_cg_product_bwd")
        return gF

    def fn_wmm_fwd(self, FF, W, stds, cnt, eps, flags):
        B = FF.shape[0]
        self.check_batch(B, FF=(FF, self.n_FF))
        self.check_weights(W, stds, flags)
        O = torch.empty(B, self.n_O, 2, device=FF.device, dtype=torch.float32)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().cgb200_fn_wmm_fwd(self.handle, _ptr(FF), _ptr(W), _ptr(stds), cnt, eps, flags, _ptr(O), B,
                                                     _stream_ptr(self.device)), "cgb200_fn_wmm_fwd")
        return O

    def fn_wmm_bwd(self, gO, FF, W, stds, eps, flags):
        self.check_batch(FF.shape[0], FF=(FF, self.n_FF), gO=(gO, self.n_O))
        self.check_weights(W, stds, flags)
        gFF = torch.empty_like(FF)
        gW = torch.empty_like(W)
        with torch.cuda.device(self.device):
            _lib.check(_lib.load().cgb200_fn_wmm_bwd(self.handle, _ptr(gO), _ptr(FF), _ptr(W), _ptr(stds), eps, flags,
                                                     _ptr(gFF), _ptr(gW), FF.shape[0], _stream_ptr(self.device)),
                       "cgb200_fn_wmm_bwd")
        return gFF, gW

    def _workspace_bytes(self, B, fwd_flags=None):
        """Workspace of the backward (``fwd_flags=None``: it also serves any forward) or of a forward with these flags.
        The size depends on the batch, the flags and the plan's options only: asked once per combination, forgotten when
        an option changes (``set_option``)."""
        key = (B, None if fwd_flags is None else fwd_flags & (_lib.FN_PRESENT | _lib.FN_UPDATE))
        n = self._ws_bytes.get(key)
        if n is None:
            lib = _lib.load()
            if fwd_flags is None:
                n = int(lib.cgb200_layer_workspace_bytes(self.handle, B))
            else:
                n = int(lib.cgb200_layer_fwd_workspace_bytes_for(self.handle, B, int(fwd_flags)))
            if n < 0:
                _lib.check(1, "cgb200_layer_workspace_bytes")
            self._ws_bytes[key] = n
        return n

    def _workspace(self, B, fwd_flags=None):
        n = self._workspace_bytes(B, fwd_flags)
        return torch.empty(max(n, 256), dtype=torch.uint8, device=self.device), n

    def _call(self, fn, name, *args):
        """Call a library entry point with this plan's device current (the per-step path of a training loop: the device
        is switched only when it is not current already)."""
        if torch.cuda.current_device() == self.device.index:
            status = fn(self.handle, *args, _current_stream(self.device.index))
        else:
            with torch.cuda.device(self.device):
                status = fn(self.handle, *args, _current_stream(self.device.index))
        if status != 0:
            _lib.check(status, name)

    def keeps_mid(self, B):
        """Does a forward with a statistics update for B samples leave the mid activation's tiles in its workspace
        (tensor-core path, tile edge 4)?  Then ``layer_fwd(..., keep=True)`` hands the workspace back and
        ``layer_bwd(..., kept=workspace)`` lets the weight gradient read the tiles instead of generating them again."""
        key = ("keeps", B)
        v = self._ws_bytes.get(key)
        if v is None:
            v = self._ws_bytes[key] = int(_lib.load().cgb200_layer_keeps_mid(self.handle, B))
        return bool(v)

    def layer_fwd(self, F, W, stds, cnt, eps, flags, keep=False):
        """``keep=True`` (only where ``keeps_mid(B)`` and with ``FN_UPDATE``): returns ``(O, workspace)``; the workspace, sized
        for the backward as well, holds the tiles and must reach ``layer_bwd`` untouched."""
        B = F.shape[0]
        self.check_batch(B, F=(F, self.n_F))
        self.check_weights(W, stds, flags)
        O = torch.empty(B, self.n_O, 2, device=self.device, dtype=torch.float32)
        ws, n = self._workspace(B, None if keep else flags)
        self._call(self._fn_layer_fwd, "cgb200_layer_fwd", F.data_ptr(), W.data_ptr(), _ptr(stds), cnt, eps, flags, O.data_ptr(),
                   B, ws.data_ptr(), n)
        return (O, ws) if keep else O

    def packed_weights_bytes(self):
        """Size of the packed form of the weights the tensor-core forward multiplies by; 0 where the forward does not use one."""
        v = self._ws_bytes.get("packed")
        if v is None:
            v = self._ws_bytes["packed"] = int(_lib.load().cgb200_layer_packed_weights_bytes(self.handle))
        return v

    def pack_weights(self, W, stds, eps, flags):
        """Pack W / max(eps, stds) once for ``layer_fwd_packed`` (inference with weights that do not change)."""
        self.check_weights(W, stds, flags)
        n = self.packed_weights_bytes()
        if n <= 0:
            raise RuntimeError("this plan's forward does not use packed weights")
        packed = torch.empty(n, dtype=torch.uint8, device=self.device)
        self._call(_lib.load().cgb200_layer_pack_weights, "cgb200_layer_pack_weights", W.data_ptr(), _ptr(stds), eps,
                   flags & _lib.FN_PRESENT, packed.data_ptr(), n)
        return packed

    def layer_fwd_packed(self, F, packed):
        """The forward of ``layer_fwd`` (stored statistics) with weights packed beforehand by ``pack_weights``: same bits."""
        B = F.shape[0]
        self.check_batch(B, F=(F, self.n_F))
        if packed.device != self.device or packed.numel() < self.packed_weights_bytes() or self.packed_weights_bytes() <= 0:
            raise RuntimeError("the packed weights do not belong to this plan")
        O = torch.empty(B, self.n_O, 2, device=self.device, dtype=torch.float32)
        ws, n = self._workspace(B, 0)
        self._call(_lib.load().cgb200_layer_fwd_packed, "cgb200_layer_fwd_packed", F.data_ptr(), packed.data_ptr(), O.data_ptr(), B,
                   ws.data_ptr(), n)
        return O

    def layer_bwd(self, F, W, stds, eps, flags, gO, need_gF=True, kept=None):
        B = F.shape[0]
        self.check_batch(B, F=(F, self.n_F), gO=(gO, self.n_O))
        self.check_weights(W, stds, flags)
        gF = torch.empty_like(F) if need_gF else None
        gW = torch.empty_like(W)
        if kept is not None:
            ws, n = kept, self._workspace_bytes(B)
            if kept.device != self.device or kept.numel() < n:
                raise RuntimeError("the kept workspace does not belong to this plan and batch")
            flags = flags | _lib.FN_KEEP_MID
        else:
            ws, n = self._workspace(B)
        self._call(self._fn_layer_bwd, "cgb200_layer_bwd", F.data_ptr(), W.data_ptr(), _ptr(stds), eps, flags, gO.data_ptr(),
                   _ptr(gF), gW.data_ptr(), B, ws.data_ptr(), n)
        return gF, gW


@functools.lru_cache(maxsize=64)
def _cached_plan(lmax, taus, tau_out, llls, device, depthwise, tile):
    return Plan(lmax, taus, tau_out, llls, device, depthwise, tile)


def get_plan(lmax, taus, tau_out, llls, device, depthwise=False, tile=0):
    """Modules with the same shape on the same device share one plan (its tables never change; its kernel-selection
    options are shared with it).  ``tile`` forces the channel-tile edge, 0 leaves the choice to the library."""
    dev = torch.device(device)
    if dev.type == "cuda" and dev.index is None:
        dev = torch.device("cuda", torch.cuda.current_device())
    return _cached_plan(int(lmax), tuple(int(t) for t in taus), None if tau_out is None else tuple(int(t) for t in tau_out),
                        tuple(int(c) for c in llls), str(dev), bool(depthwise), int(tile))


# ----------------------------------------------------------------------------------------------------------------
# CG table helpers with the reference's names
# ----------------------------------------------------------------------------------------------------------------
def _precomputeCG_cuda(lmax, llls, device="cuda"):
    """CG band table and its offsets as device tensors (reference: ``CG_layers.py:134-141``)."""
    lib = _lib.load()
    dev = torch.device(device)
    offsets = CGutils.SparseLtuples.cal_CG_offsets(lmax, llls)
    CG_coefs = torch.empty(offsets[-1], dtype=torch.float, device=dev)
    a_l = _lib.i32(llls)
    with torch.cuda.device(dev):
        _lib.check(lib.cgb200_cg_table_build(_ptr(CG_coefs), offsets[-1], lmax, a_l, len(llls), _stream_ptr(dev)),
                   "cgb200_cg_table_build")
    return CG_coefs, torch.tensor(offsets, dtype=torch.int, device=dev)


def _precomputeCG_MST(lmax, method="mst", device="cuda"):
    assert method == "mst", "%s is not implemented" % method
    llls = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(CGutils.SparseLtuples.compute_mst_ltuples(lmax))[0]
    return _precomputeCG_cuda(lmax, llls, device)


@functools.lru_cache(10)
def precomputeCG(lmax, method="mst", device="cuda"):
    """Cached CG table for the full (``method=None``) or MST pair lists (reference: ``CG_layers.py:153-165``)."""
    if method is None:
        llls = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(CGutils.SparseLtuples.compute_default_ltuples(lmax))[0]
        return _precomputeCG_cuda(lmax, llls, device)
    if method == "mst":
        return _precomputeCG_MST(lmax, "mst", device)
    raise NotImplementedError()


# ----------------------------------------------------------------------------------------------------------------
# autograd glue
# ----------------------------------------------------------------------------------------------------------------
class _CG_sparse_cuda(torch.autograd.Function):
    """Product forward/backward (reference: ``CG_layers.py:168-203``)."""

    @staticmethod
    def forward(ctx, Fs, plan):
        Fs = _check_cuda_f32(Fs, "activations")
        ctx.plan = plan
        ctx.save_for_backward(Fs)
        return plan.cg_product_fwd(Fs)

    @staticmethod
    def backward(ctx, grad_output):
        (Fs,) = ctx.saved_tensors
        return ctx.plan.cg_product_bwd(Fs, _check_cuda_f32(grad_output, "grad_output")), None


def _fn_flags(bn_stds, update):
    flags = 0
    if bn_stds is not None:
        flags |= _lib.FN_PRESENT
        if update:
            flags |= _lib.FN_UPDATE
    return flags


class _MyBatchNormWeightMM_cuda(torch.autograd.Function):
    """Norm + mixing forward/backward on a materialised product (reference: ``CG_layers.py:14-72``).  As there, the
    forward updates ``bn_stds`` in place when asked to and the backward uses the updated values."""

    @staticmethod
    def forward(ctx, FF, W, plan, bn_stds, bn_cnt, bn_eps, bn_updateflag):
        FF = _check_cuda_f32(FF, "FF")
        W = _check_cuda_f32(W, "W")
        flags = _fn_flags(bn_stds, bn_updateflag)
        out = plan.fn_wmm_fwd(FF, W, bn_stds, float(bn_cnt), float(bn_eps), flags)
        ctx.plan, ctx.eps, ctx.flags = plan, float(bn_eps), flags & _lib.FN_PRESENT
        ctx.save_for_backward(FF, W, None if bn_stds is None else bn_stds.detach().clone())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        FF, W, stds = ctx.saved_tensors
        gFF, gW = ctx.plan.fn_wmm_bwd(_check_cuda_f32(grad_output, "grad_output"), FF, W, stds, ctx.eps, ctx.flags)
        return gFF, gW, None, None, None, None, None


# bytes of layer workspaces currently kept for a backward, per device, and the devices' memory sizes
_kept_bytes = {}
_device_bytes = {}


def _note_kept(ws):
    """Account for a kept workspace until its tensor is released (after the backward, or when the graph is dropped)."""
    dev, n = ws.device, ws.numel()
    _kept_bytes[dev] = _kept_bytes.get(dev, 0) + n

    def release():
        _kept_bytes[dev] = _kept_bytes.get(dev, 0) - n
    weakref.finalize(ws, release)


class _CGBN_fused(torch.autograd.Function):
    """Whole layer through the fused kernels: the mid activation is regenerated in the backward, never stored."""

    @staticmethod
    def forward(ctx, Fs, W, plan, bn_stds, bn_cnt, bn_eps, bn_updateflag, keep_mid=False):
        Fs = _check_cuda_f32(Fs, "activations")
        W = _check_cuda_f32(W, "W")
        flags = _fn_flags(bn_stds, bn_updateflag)
        ctx.kept = None
        if keep_mid and (flags & _lib.FN_UPDATE) and plan.keeps_mid(Fs.shape[0]):
            out, ctx.kept = plan.layer_fwd(Fs, W, bn_stds, float(bn_cnt), float(bn_eps), flags, keep=True)
            _note_kept(ctx.kept)
        else:
            out = plan.layer_fwd(Fs, W, bn_stds, float(bn_cnt), float(bn_eps), flags)
        ctx.plan, ctx.eps, ctx.flags = plan, float(bn_eps), flags & _lib.FN_PRESENT
        ctx.save_for_backward(Fs, W, None if bn_stds is None else bn_stds.detach().clone())
        return out

    @staticmethod
    def backward(ctx, grad_output):
        Fs, W, stds = ctx.saved_tensors
        kept, ctx.kept = ctx.kept, None   # one backward per forward: the workspace is overwritten by it
        gF, gW = ctx.plan.layer_bwd(Fs, W, stds, ctx.eps, ctx.flags, _check_cuda_f32(grad_output, "grad_output"),
                                    need_gF=ctx.needs_input_grad[0], kept=kept)
        return gF, gW, None, None, None, None, None, None


# ----------------------------------------------------------------------------------------------------------------
# modules
# ----------------------------------------------------------------------------------------------------------------
def _flatten_input(activations):
    if isinstance(activations, (list, tuple)):
        B = activations[0].shape[0]
        return torch.cat([v.reshape(B, -1, 2) for v in activations], dim=1)
    return activations


class MyBatchNormWeightMM_cuda(nn.Module):
    """Fragment norm and per-degree mixing weights (reference: ``CG_layers.py:74-132``).

    Parameters: ``W`` flat ``(sum_l t_FF[l]*tau_out[l], 2)`` = ``weight_scale * U[0,1)``; ``bn_stds`` flat
    ``(sum_l t_FF[l],)`` = ``U[0,1)`` (``None`` without batchnorm), not trainable; ``bn_eps`` ``(1,)``.  ``init='debug'``
    seeds torch and numpy with 0 first, as the reference does.
    """

    def __init__(self, lmax, t_FF, tau_out, batchnorm=True, weight_scale=0.05, init="random", eps=1e-5, device="cuda",
                 plan=None):
        super().__init__()
        self.lmax = lmax
        self._init_method = init
        self.weight_scale = weight_scale
        self.t_FF = np.asarray(t_FF)
        assert len(self.t_FF) - 1 == lmax
        self.t_O = tau_out
        m = 1 + 2 * np.arange(lmax + 1)
        self.cumu_tm_FF = np.concatenate([[0], (self.t_FF * m).cumsum()])
        self.cumu_tm_O = np.concatenate([[0], (np.asarray(tau_out) * m).cumsum()])
        self.cumu_tm_W = np.concatenate([[0], (self.t_FF * np.asarray(tau_out)).cumsum()])
        self.batchnorm = batchnorm
        self.bn_stds = None
        self.bn_eps = nn.Parameter(eps * torch.ones(1), requires_grad=False)
        self._eps = float(eps)
        self.register_buffer("bn_cnt_buf", torch.ones(1, dtype=torch.float64))
        self.W = None
        self._device = torch.device(device)
        self.reset_parameters()
        self._plan = plan   # set by CGBN_cuda; a stand-alone module builds a mixing-only plan lazily
        self.to(device)

    @property
    def bn_cnt(self):
        return self._count()

    @bn_cnt.setter
    def bn_cnt(self, v):
        self._cnt_cache = float(v)
        self.bn_cnt_buf.fill_(float(v))

    def _save_to_state_dict(self, destination, prefix, keep_vars):
        # the counter lives on the host between checkpoints (one device write per layer and step saved); the buffer is
        # brought up to date when a state dict is taken
        if getattr(self, "_cnt_cache", None) is not None:
            self.bn_cnt_buf.fill_(self._cnt_cache)
        super()._save_to_state_dict(destination, prefix, keep_vars)

    def _load_from_state_dict(self, state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs):
        # checkpoints written by the reference have no counter: keep the current one instead of failing
        key = prefix + "bn_cnt_buf"
        if key not in state_dict:
            if getattr(self, "_cnt_cache", None) is not None:
                self.bn_cnt_buf.fill_(self._cnt_cache)
            state_dict[key] = self.bn_cnt_buf.detach().clone()
        super()._load_from_state_dict(state_dict, prefix, local_metadata, strict, missing_keys, unexpected_keys, error_msgs)
        self._cnt_cache = None
        # the kernels take eps as a host float: follow the checkpoint's value (the reference passes the parameter itself)
        self._eps = float(self.bn_eps.detach().cpu().item())

    def reset_parameters(self):
        if self._init_method not in {"debug", "random"}:
            raise NotImplementedError()
        if self._init_method == "debug":
            torch.manual_seed(0)
            np.random.seed(0)
        if self.batchnorm:
            std_flat_np = np.random.rand(int(np.sum(self.t_FF)))
            self.bn_stds = nn.Parameter(torch.tensor(std_flat_np, dtype=torch.float), requires_grad=False)
        wlength = int(np.sum(self.t_FF * np.asarray(self.t_O)))
        wbig = self.weight_scale * torch.rand(wlength, 2, device=self._device, dtype=torch.float)
        self.W = nn.Parameter(wbig, requires_grad=True)
        self._cnt_cache = 1.0

    def _count(self):
        # the counter is read on the host every training step; keep a host copy so the buffer needs no device sync
        if getattr(self, "_cnt_cache", None) is None:
            self._cnt_cache = float(self.bn_cnt_buf.item())
        return self._cnt_cache

    def _bump(self):
        self._cnt_cache = self._count() + 1.0

    def _mix_plan(self):
        if self._plan is None:
            # Stand-alone use: mixing never looks at the pairs, only at the channel counts.  A depthwise plan with one
            # pseudo-triple (l, l, l) per degree and tau_in = t_FF reproduces exactly those counts.
            L1 = self.lmax + 1
            llls = [(l * L1 + l) * L1 + l for l in range(L1) if self.t_FF[l] > 0]
            self._plan = get_plan(self.lmax, self.t_FF, self.t_O, llls, self.W.device, depthwise=True)
            assert self._plan.t_ff() == [int(t) for t in self.t_FF]
        return self._plan

    def forward(self, FF):
        update = bool(self.batchnorm and self.training)
        out = _MyBatchNormWeightMM_cuda.apply(FF, self.W, self._mix_plan(), self.bn_stds, self._count(), self._eps, update)
        if update:
            self._bump()
        return out


class CG_woFilter_cuda(nn.Module):
    """The CG product of an activation with itself (reference: ``CG_layers.py:205-286``).

    ``lll_mode``: ``None`` (all pairs), ``'mst'``, ``'debug'`` or an explicit per-degree list of ``(l1, l2)`` lists.
    """

    def __init__(self, lmax, taus, lll_mode=None, device="cuda", tau_out=None, depthwise=False):
        super().__init__()
        self.lmax = lmax
        self.t_F = taus
        self.cum_taus = CGutils.cumulative_tm(taus)
        self._device = torch.device(device)
        if lll_mode is None:
            ltuples = CGutils.SparseLtuples.compute_default_ltuples(lmax)
        elif isinstance(lll_mode, str) and lll_mode == "mst":
            ltuples = CGutils.SparseLtuples.compute_mst_ltuples(lmax)
        elif isinstance(lll_mode, str) and lll_mode == "debug":
            ltuples = CGutils.SparseLtuples.compute_debug_ltuples(lmax)
        else:
            ltuples = lll_mode
        self.lll_mode = lll_mode if (lll_mode is None or isinstance(lll_mode, str)) else "custom"
        self.depthwise = bool(depthwise)
        self.lll_list, self.l_l1_to_lllidx_offsets = CGutils.SparseLtuples.sparse_rep_ltuples_sorted(ltuples)
        self.t_FF, self._t_offsets = CGutils.SparseLtuples.cal_new_tau_and_offsets(lmax, taus, self.lll_list, depthwise)
        self.cumu_tm_FF = CGutils.cumulative_tm(self.t_FF)
        self.plan = get_plan(lmax, taus, tau_out, self.lll_list, device, depthwise)
        assert self.plan.t_ff() == [int(t) for t in self.t_FF], "host and library disagree on the mid-channel counts"
        self._cg_cache = None

    # CG table as tensors, for callers that look at them (the kernels use the plan's resident copy)
    def _cg_tensors(self):
        if self._cg_cache is None:
            if self.lll_mode is None or self.lll_mode == "mst":
                self._cg_cache = precomputeCG(self.lmax, self.lll_mode, str(self.plan.device))
            else:
                self._cg_cache = _precomputeCG_cuda(self.lmax, self.lll_list, device=self.plan.device)
        return self._cg_cache

    @property
    def CGspace(self):
        return self._cg_tensors()[0]

    @property
    def CG_offsets(self):
        return self._cg_tensors()[1]

    def cal_new_tau_and_offsets(self, taus):
        return CGutils.SparseLtuples.cal_new_tau_and_offsets(self.lmax, taus, self.lll_list, self.depthwise)

    def forward(self, activations, straight_output=True):
        new_activations = _flatten_input(activations)
        if not new_activations.is_cuda:
            raise RuntimeError("activations must be CUDA tensors (cgnet_b200 has no CPU path)")
        output = _CG_sparse_cuda.apply(new_activations, self.plan)
        if not straight_output:
            output = CGutils.reshape_out(output, self.t_FF)
        return output


class CGBN_cuda(nn.Module):
    """One CG layer: product, fragment norm, mixing (reference: ``CG_layers.py:289-318``).

    ``forward(fs, straight_output=False)`` takes a list of ``(B, tau_l, 2l+1, 2)`` tensors or the flat
    ``(B, sum_l tau_l(2l+1), 2)`` tensor and returns a list (default) or the flat tensor.
    """

    def __init__(self, lmax, taus_fs, tau_out, batchnorm=True, sparse_flag=False, device="cuda", weight_scale=0.05,
                 init="random", eps=1e-5, fused=True, depthwise=False, lll_mode=None, keep_mid=None):
        super().__init__()
        self.lmax = lmax
        self._init_method = init
        self.sparse_flag = sparse_flag
        self.fused = fused
        self.keep_mid = keep_mid
        self.pack_inference_weights = True
        self._packed, self._packed_key = None, None
        mode = lll_mode if lll_mode is not None else ("mst" if sparse_flag else None)
        self.cg = CG_woFilter_cuda(lmax, taus_fs, lll_mode=mode, device=device, tau_out=tau_out, depthwise=depthwise)
        self.t_F = self.cg.t_F
        self.t_FF = self.cg.t_FF
        self.tau_out = tau_out
        self.bnWMM = MyBatchNormWeightMM_cuda(lmax, self.t_FF, tau_out, batchnorm, weight_scale, init, eps, device,
                                              plan=self.cg.plan)
        self.to(device)

    def _packed_weights(self):
        """Inference without autograd on the tensor-core path: the packed form of W / max(eps, stds) is built once and
        reused until W, the statistics, eps or the plan's options change (``pack_inference_weights=False`` switches the
        cache off; it holds as many bytes again as four times the weights)."""
        bn, plan = self.bnWMM, self.cg.plan
        if not self.pack_inference_weights or plan.packed_weights_bytes() <= 0:
            return None
        stds = bn.bn_stds if bn.batchnorm else None
        key = (bn.W.data_ptr(), bn.W._version, None if stds is None else (stds.data_ptr(), stds._version), bn._eps, bn._count(),
               plan.packed_weights_bytes(), plan._option_epoch)
        if self._packed_key != key:
            self._packed = plan.pack_weights(bn.W.detach(), None if stds is None else stds.detach(), bn._eps,
                                             _lib.FN_PRESENT if stds is not None else 0)
            self._packed_key = key
        return self._packed

    def _keeps_mid(self, B):
        """Keep the layer's workspace from the forward to the backward, so that the weight gradient reads the mid
        activation's tiles the forward left in it instead of generating them again (wide layers on the tensor-core path
        only: ``Plan.keeps_mid``)?  ``keep_mid=True`` / ``False`` decide; the default keeps workspaces of 64 MB and more while
        the workspaces kept on the device at that moment (by all layers: each is held until its layer's backward has run),
        this one included, stay under a quarter of the device's memory."""
        if self.keep_mid is False:
            return False
        plan = self.cg.plan
        if not plan.keeps_mid(B):
            return False
        if self.keep_mid:
            return True
        need = plan._workspace_bytes(B)
        if need < (64 << 20):
            return False   # a small layer: what the kept tiles save on the GPU is less than the host time of keeping them
        dev = plan.device
        if dev not in _device_bytes:
            _device_bytes[dev] = torch.cuda.get_device_properties(dev).total_memory
        return (_kept_bytes.get(dev, 0) + need) * 4 <= _device_bytes[dev]

    def forward(self, fs, straight_output=False):
        bn = self.bnWMM
        if self.fused:
            x = _flatten_input(fs)
            update = bool(bn.batchnorm and bn.training)
            if not update and not torch.is_grad_enabled():
                packed = self._packed_weights()
                if packed is not None:
                    new_fs = self.cg.plan.layer_fwd_packed(_check_cuda_f32(x, "activations"), packed)
                    return new_fs if straight_output else CGutils.reshape_out(new_fs, self.tau_out)
            keep = update and torch.is_grad_enabled() and self._keeps_mid(x.shape[0])
            new_fs = _CGBN_fused.apply(x, bn.W, self.cg.plan, bn.bn_stds, bn._count(), bn._eps, update, keep)
            if update:
                bn._bump()
        else:
            new_fs = bn(self.cg(fs, straight_output=True))
        if not straight_output:
            new_fs = CGutils.reshape_out(new_fs, self.tau_out)
        return new_fs
