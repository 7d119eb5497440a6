"""CPU oracle for the Clebsch-Gordan layer.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline / reference legs of ``bench.py`` may import this
module; nothing under ``cgnet_b200/`` does.  It restates, on the CPU, what the reference project (zlin7/CGNet)
computes on the path  CG product -> fragment-norm scale -> per-degree complex channel mixing.  Each function names
the reference lines it follows (paths are relative to the reference checkout).

Pinning: ``tests/golden/make_golden.py`` imported the reference's own Python path (``CGNet/CG_layers_python.py`` with
its compiled ``ClebschGordan`` module) on a CPU and stored its index tables, CG matrices, layer outputs and autograd
gradients as fixtures; ``tests/test_oracle.py`` checks every function here against those fixtures.  The training-mode
fragment-norm statistics are the one piece the reference cannot execute without a GPU (its twin calls ``.cuda()``
inside, ``CG_layers_python.py:177``); that piece is pinned by a numpy transcription of lines 175-179 made inside the
fixture script.

Conventions (all from the reference):
  * activation ``float[B][N][2]``, fragment l at ``cum[l] = sum_{l'<l} tau_l'(2l'+1)``, inner index ``t(2l+1)+(m+l)``,
    last axis (re, im)   (``CGNet/CGutils.py:190-197``, ``CGNet/cudaCG/cudaCG_sparse.cu:17``);
  * triples ``(l, l1, l2)`` with ``l2 <= l1``, ordered by l then (stably) by l1, encoded ``(l(L+1)+l1)(L+1)+l2``
    (``CGNet/CGutils.py:122-140``);
  * mid channel of triple k inside degree l: ``t_offsets[k] + t1*tau_l2 + t2`` (``CGNet/CG_layers.py:253-262``);
  * mixing weights flat ``(sum_l t_FF[l]*tau_out[l], 2)``, per degree row-major ``(tau_out[l], t_FF[l])``
    (``CGNet/CG_layers.py:98``, ``CGNet/cudaCG/cudaCG_FNWMM.cu:18``).
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from functools import lru_cache

import numpy as np
import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def _lib():
    """Load (building on first use) the plain-C coefficient oracle ``oracle/cg_coeff_oracle.c``."""
    global _LIB
    if _LIB is None:
        so = os.path.join(_HERE, "_build", "libcg_oracle.so")
        src = os.path.join(_HERE, "cg_coeff_oracle.c")
        if not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
            os.makedirs(os.path.dirname(so), exist_ok=True)
            subprocess.check_call(["gcc", "-O2", "-fPIC", "-shared", "-o", so, src, "-lm"])
        lib = ctypes.CDLL(so)
        lib.cg_oracle_coeff.restype = ctypes.c_double
        lib.cg_oracle_coeff.argtypes = [ctypes.c_int] * 5
        lib.cg_oracle_dense.restype = None
        lib.cg_oracle_dense.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p]
        lib.cg_oracle_band.restype = None
        lib.cg_oracle_band.argtypes = [ctypes.c_int] * 3 + [ctypes.c_void_p]
        _LIB = lib
    return _LIB


# --------------------------------------------------------------------------------------------------------------------
# Clebsch-Gordan coefficients
# --------------------------------------------------------------------------------------------------------------------
def cg_coeff(l1, l2, l, m1, m2):
    """<l1 m1; l2 m2 | l m1+m2>, double.  Follows ``ClebschGordan.cpp:360-394`` / ``cudaCG_sparse.cu:33-57``."""
    return float(_lib().cg_oracle_coeff(l1, l2, l, m1, m2))


@lru_cache(maxsize=None)
def cg_dense(l1, l2, l):
    """Dense ``(2l+1, (2l1+1)(2l2+1))`` float64 matrix, column ``(m1+l1)(2l2+1)+(m2+l2)`` (``CGmodule.cpp:85-99``)."""
    out = np.zeros((2 * l + 1, (2 * l1 + 1) * (2 * l2 + 1)), dtype=np.float64)
    _lib().cg_oracle_dense(l1, l2, l, out.ctypes.data)
    return out


def cg_band_table(lmax, llls):
    """Flat fp32 band table + offsets: per triple ``(2l+1) x (2l2+1)``, entry ``[m+l][m2+l2]`` with ``m1 = m-m2``.

    Layout of the reference's device table (``cudaCG_sparse.cu:68-92``) and of its CPU builder
    (``CGutils.py:161-177``); offsets as ``CGutils.py:180-187``.
    """
    offs = cg_offsets(lmax, llls)
    out = np.zeros(offs[-1], dtype=np.float32)
    for k, (l, l1, l2) in enumerate(decode_triples(lmax, llls)):
        _lib().cg_oracle_band(l1, l2, l, out[offs[k]:].ctypes.data)
    return out, np.asarray(offs, dtype=np.int64)


# --------------------------------------------------------------------------------------------------------------------
# Index layer: which (l1, l2) pairs feed each output degree, and where every channel lives
# --------------------------------------------------------------------------------------------------------------------
def default_ltuples(lmax):
    """All pairs ``l2 <= l1 <= lmax`` per admissible l (``CGutils.py:113-119``)."""
    out = [[] for _ in range(lmax + 1)]
    for l1 in range(lmax + 1):
        for l2 in range(l1 + 1):
            for l in range(l1 - l2, min(l1 + l2, lmax) + 1):
                out[l].append((l1, l2))
    return out


def debug_ltuples(lmax):
    """First two admissible pairs per l in the default enumeration order (``CGutils.py:103-110``)."""
    return [pairs[:2] for pairs in default_ltuples(lmax)]


def mst_pairs(l, lmax, diag=True):
    """Minimum-spanning-tree pair selection for one output degree (``CGutils.py:73-98``).

    Nodes are the degrees 0..lmax; an edge joins a < b when ``b-a <= l <= a+b`` with weight (2l+1)(2a+1)(2b+1).  The
    edge is stored at (row b, col a), so the tree comes back with the larger degree first.  Every diagonal pair
    (a, a) with ``l <= 2a`` is appended.  scipy's tie-breaking decides between equal-weight trees, exactly as in the
    reference, which calls the same routine.
    """
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import minimum_spanning_tree

    rows, cols, w = [], [], []
    for a in range(lmax + 1):
        for b in range(a + 1, lmax + 1):
            if b - a <= l <= a + b:
                rows.append(b)
                cols.append(a)
                w.append((2 * l + 1) * (2 * a + 1) * (2 * b + 1))
    tree = minimum_spanning_tree(csr_matrix((w, (rows, cols)), shape=(lmax + 1, lmax + 1))).tocoo()
    pairs = list(zip(tree.row.tolist(), tree.col.tolist()))
    if diag:
        pairs += [(a, a) for a in range(lmax + 1) if l <= 2 * a]
    return pairs


def mst_ltuples(lmax):
    """Per-l MST pair lists with the diagonal added (``CG_layers.py:143-151``, ``CG_layers_python.py:82-86``)."""
    return [mst_pairs(l, lmax, diag=True) for l in range(lmax + 1)]


def encode_sorted(ltuples):
    """Canonical triple list and the (L+1)x(L+2) cumulative (l, l1) -> triple-index table (``CGutils.py:122-140``)."""
    lmax = len(ltuples) - 1
    L1 = lmax + 1
    llls = []
    counts = np.zeros((L1, L1), dtype=np.int64)
    for l in range(L1):
        pairs = sorted(ltuples[l], key=lambda p: p[0])  # stable: ties keep their incoming order
        for l1, l2 in pairs:
            assert l1 >= l2, "pairs must come with l2 <= l1"
            llls.append((l * L1 + l1) * L1 + l2)
            counts[l, l1] += 1
    table = np.zeros((L1, L1 + 1), dtype=np.int64)
    start = 0
    for l in range(L1):
        table[l, 0] = start
        table[l, 1:] = start + np.cumsum(counts[l])
        start = table[l, -1]
    return llls, table.reshape(-1)


def decode_triples(lmax, llls):
    """``[(l, l1, l2), ...]`` from the encoded list (``CGutils.py:143-151``)."""
    L1 = lmax + 1
    return [(c // (L1 * L1), (c // L1) % L1, c % L1) for c in llls]


def cg_offsets(lmax, llls):
    """Start of each triple's band table, plus the total length (``CGutils.py:180-187``)."""
    offs = [0]
    for l, _, l2 in decode_triples(lmax, llls):
        offs.append(offs[-1] + (2 * l + 1) * (2 * l2 + 1))
    return offs


def tau_ff_and_offsets(lmax, taus, llls):
    """Mid-channel count per degree and first mid channel of every triple (``CG_layers.py:253-262``)."""
    t_ff = np.zeros(lmax + 1, dtype=np.int64)
    offs = []
    for l, l1, l2 in decode_triples(lmax, llls):
        offs.append(int(t_ff[l]))
        t_ff[l] += taus[l1] * taus[l2]
    return t_ff, offs


def cumulative_tm(taus):
    """``cum[l] = sum_{l'<l} taus[l'] (2l'+1)`` with the total appended (``CG_layers.py:219``)."""
    taus = np.asarray(taus, dtype=np.int64)
    return np.concatenate([[0], np.cumsum(taus * (2 * np.arange(len(taus)) + 1))])


def split_fragments(flat, taus):
    """Flat ``(B, N, 2)`` -> list of ``(B, tau_l, 2l+1, 2)`` views (``CGutils.py:190-197``)."""
    out, off = [], 0
    for l, t in enumerate(taus):
        n = (2 * l + 1) * int(t)
        out.append(flat[:, off:off + n, :].reshape(flat.shape[0], int(t), 2 * l + 1, 2))
        off += n
    assert off == flat.shape[1]
    return out


def join_fragments(frags):
    """List of ``(B, tau_l, 2l+1, 2)`` -> flat ``(B, N, 2)`` (``CG_layers.py:275``)."""
    B = frags[0].shape[0]
    return torch.cat([f.reshape(B, -1, 2) for f in frags], dim=1)


# --------------------------------------------------------------------------------------------------------------------
# The layer, piece by piece (torch on CPU so that autograd supplies the reference's gradients)
# --------------------------------------------------------------------------------------------------------------------
def _as_complex(x):
    return torch.view_as_complex(x.contiguous())


def cg_product(frags, taus, lmax, llls, depthwise=False):
    """CG product of a fragment list with itself over the given triples.

    Follows ``CG_sparse_py.forward`` (``CG_layers_python.py:113-133``): for a triple, form the Kronecker product of
    fragment l1 and fragment l2 over both the m and the channel axes (``Complex_math.py:12-35``: row (m1, m2), column
    t1*tau_l2 + t2), multiply from the left by the dense CG matrix (``CG_layers_python.py:106-111``) and append the
    result to degree l in triple order.  Returns a list of ``(B, t_FF[l], 2l+1, 2)``; an empty degree gets 0 channels.

    ``depthwise=True`` keeps only t1 == t2 (needs tau_l1 == tau_l2).  The reference has no such product: that mode is
    an extension whose parity is unpinned.
    """
    B = frags[0].shape[0]
    dtype = frags[0].dtype
    cdt = torch.complex64 if dtype == torch.float32 else torch.complex128
    z = [_as_complex(f) for f in frags]                      # (B, tau, 2l+1)
    out = [[] for _ in range(lmax + 1)]
    for l, l1, l2 in decode_triples(lmax, llls):
        C = torch.from_numpy(cg_dense(l1, l2, l)).to(dtype).to(cdt)               # (2l+1, n1*n2)
        if depthwise:
            assert taus[l1] == taus[l2]
            kp = z[l1].unsqueeze(3) * z[l2].unsqueeze(2)                          # (B, t, m1, m2)
            kp = kp.reshape(B, taus[l1], (2 * l1 + 1) * (2 * l2 + 1))
        else:
            kp = z[l1][:, :, None, :, None] * z[l2][:, None, :, None, :]          # (B, t1, t2, m1, m2)
            kp = kp.reshape(B, taus[l1] * taus[l2], (2 * l1 + 1) * (2 * l2 + 1))
        out[l].append(torch.matmul(kp, C.t()))                                     # (B, t1*t2, 2l+1)
    res = []
    for l in range(lmax + 1):
        if out[l]:
            res.append(torch.view_as_real(torch.cat(out[l], dim=1)))
        else:
            res.append(torch.zeros(B, 0, 2 * l + 1, 2, dtype=dtype))
    return res


def fragment_norm_stats(ff_frags):
    """Per mid channel: std over (batch, m) of the complex modulus, ddof=0, in float64.

    ``CG_layers_python.py:175-177`` (``np.linalg.norm`` over the re/im axis, then ``np.std`` over axes (0, 2));
    the CUDA path computes sqrt(E|z|^2 - (E|z|)^2) in double (``cudaCG_FNWMM.cu:55-74``), the same quantity.
    """
    sig = []
    for f in ff_frags:
        a = f.detach().to(torch.float64).numpy()
        if a.shape[1] == 0:
            continue
        sig.append(np.std(np.linalg.norm(a, ord=2, axis=3), axis=(0, 2)))
    return np.concatenate(sig) if sig else np.zeros(0)


def fragment_norm_update(stds, sigma, cnt):
    """Moving average ``stds*cnt/(cnt+1) + sigma/(cnt+1)`` with fp32 storage (``CG_layers_python.py:178-179``,
    ``cudaCG_FNWMM.cu:75-76``).  Returns a new float32 array."""
    s = np.asarray(stds, dtype=np.float32) * np.float32(np.float32(cnt) / np.float32(cnt + 1.0))
    return (s.astype(np.float64) + np.asarray(sigma, dtype=np.float64) / np.float64(np.float32(cnt + 1.0))).astype(np.float32)


def fragment_norm_apply(ff_frags, stds, eps):
    """Divide every mid channel by ``max(eps, std)`` (``CG_layers_python.py:181``, ``cudaCG_FNWMM.cu:112-116``)."""
    out, off = [], 0
    for f in ff_frags:
        t = f.shape[1]
        d = torch.clamp(torch.as_tensor(stds[off:off + t], dtype=f.dtype), min=float(eps)).view(1, t, 1, 1)
        out.append(f / d)
        off += t
    return out


def mix(ff_frags, W, tau_out):
    """Per-degree complex channel mixing ``O_l = W_l @ FF_l`` (``CG_layers_python.py:261-266``, ``CGutils.py:15-21``)."""
    out, off = [], 0
    for l, f in enumerate(ff_frags):
        k, to = f.shape[1], int(tau_out[l])
        Wl = _as_complex(W[off:off + k * to].reshape(to, k, 2))
        off += k * to
        out.append(torch.view_as_real(torch.matmul(Wl, _as_complex(f))))
    assert off == W.shape[0]
    return out


def cgbn_layer(frags, taus, tau_out, lmax, llls, W, stds=None, eps=1e-5, cnt=1.0, training=False, depthwise=False):
    """One full layer: CG product, optional fragment norm (with the in-place moving-average update when training),
    mixing.  Mirrors ``CGBN_base.forward`` (``CG_layers_python.py:248-269``) == ``CGBN_cuda.forward``
    (``CG_layers.py:313-318``).  Returns ``(out_frags, new_stds or None)``.  As in the reference, the statistics carry
    no gradient."""
    ff = cg_product(frags, taus, lmax, llls, depthwise=depthwise)
    new_stds = None
    if stds is not None:
        new_stds = np.asarray(stds, dtype=np.float32)
        if training:
            new_stds = fragment_norm_update(new_stds, fragment_norm_stats(ff), cnt)
        ff = fragment_norm_apply(ff, new_stds, eps)
    return mix(ff, W, tau_out), new_stds


# --------------------------------------------------------------------------------------------------------------------
# The reference's CPU algorithm with its own cost profile (materialised Kronecker products, one small bmm per triple on
# split re/im tensors): this is what the CPU-baseline leg of the benchmark times.
# --------------------------------------------------------------------------------------------------------------------
def twin_forward(frags, taus, tau_out, lmax, llls, W, stds=None, eps=1e-5, training=False, cnt=1.0):
    """Forward of one layer done the way ``CG_layers_python.py`` does it (torch ops, so autograd gives the backward
    with the same cost profile).  With ``training=True`` the fragment-norm statistics are first folded into a copy of
    ``stds`` as ``MyBatchNormList.forward`` does (``CG_layers_python.py:172-179``) and ``(out, new_stds)`` is returned.

    Per triple, repeat-materialised
    Kronecker product on separate real/imaginary tensors (``Complex_math.py:12-35,46-63``), batched matmul with the
    dense CG matrix repeated over the batch (``CG_layers_python.py:106-111``), concatenation per degree, division by
    max(eps, std), then ``Complex_bmm`` with the weights repeated over the batch (``CGutils.py:15-21``)."""
    B = frags[0].shape[0]
    fs = [f.permute(0, 2, 1, 3) for f in frags]               # (B, 2l+1, tau, 2) as the twin does
    new = [[] for _ in range(lmax + 1)]

    def kron(a, b):                                           # a: (B, n1, d1)  b: (B, n2, d2) -> (B, n1*n2, d1*d2)
        n1, d1 = a.shape[1], a.shape[2]
        n2, d2 = b.shape[1], b.shape[2]
        return a.unsqueeze(3).unsqueeze(4).repeat(1, 1, n2, d2, 1).view(B, n1 * n2, -1) * b.repeat(1, n1, d1)

    for l, l1, l2 in decode_triples(lmax, llls):
        ar, ai = fs[l1][..., 0], fs[l1][..., 1]
        br, bi = fs[l2][..., 0], fs[l2][..., 1]
        kr = kron(ar, br) - kron(ai, bi)
        ki = kron(ar, bi) + kron(ai, br)
        C = torch.from_numpy(cg_dense(l1, l2, l)).to(kr.dtype).repeat(B, 1, 1)
        new[l].append(torch.stack([torch.bmm(C, kr), torch.bmm(C, ki)], 3).permute(0, 2, 1, 3))
    ff = [torch.cat(v, 1) for v in new]
    new_stds = None
    if stds is not None:
        new_stds = np.asarray(stds, dtype=np.float32)
        if training:
            new_stds = fragment_norm_update(new_stds, fragment_norm_stats(ff), cnt)
        ff = fragment_norm_apply(ff, new_stds, eps)
    out, off = [], 0
    for l, f in enumerate(ff):
        k, to = f.shape[1], int(tau_out[l])
        wl = W[off:off + k * to].view(to, k, 2).repeat(B, 1, 1, 1)
        off += k * to
        wr, wi = wl[..., 0], wl[..., 1]
        fr, fi = f[..., 0], f[..., 1]
        out.append(torch.stack([torch.bmm(wr, fr) - torch.bmm(wi, fi), torch.bmm(wr, fi) + torch.bmm(wi, fr)], 3))
    return (out, new_stds) if training else out
