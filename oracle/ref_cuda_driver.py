"""Driver of the reference project's own CUDA extension (`CG_cuda_ops`, CGNet/cudaCG, unmodified sources compiled
for sm_100a by oracle/build_ref_cuda.py into oracle/_ref/cuda_build/).

TEST AND MEASUREMENT INFRASTRUCTURE ONLY: the GPU-side parity oracle of tests/ and the "kernel to beat" that bench.py
times beside the product.  Nothing under cgnet_b200/ imports this file or loads that module.

The reference's Python layer (CGNet/CG_layers.py) needs its C++ coefficient module and a debugger package at import
time, so it is not imported; instead the six extension functions are called directly with index tensors laid out
exactly as its modules build them (CG_layers.py:244-250 for the product, :104-108 for the mixing) and in the order its
autograd functions call them (CG_layers.py:16-72, 171-203): zero-filled outputs allocated on every call, the product
materialised, statistics updated in place by the forward, a clone of them kept for the backward.
"""
import importlib.util
import os

import numpy as np
import torch

import cg_oracle as o

HERE = os.path.dirname(os.path.abspath(__file__))
REF_SO = os.path.join(HERE, "_ref", "cuda_build", "CG_cuda_ops.so")


def available():
    return os.path.exists(REF_SO)


_ops = None


def load_ops():
    """The compiled reference extension (a pybind11 module exposing the six functions of cudaCG_all.cpp:207-215)."""
    global _ops
    if _ops is None:
        if not available():
            raise RuntimeError("reference CUDA extension not built (python oracle/build_ref_cuda.py --ref <checkout>)")
        spec = importlib.util.spec_from_file_location("CG_cuda_ops", REF_SO)
        mod = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(mod)
        _ops = mod
    return _ops


class RefLayer:
    """The index tensors of CG_woFilter_cuda / MyBatchNormWeightMM_cuda and thin calls into the reference kernels."""

    def __init__(self, ops, lmax, taus, tau_out, llls, device):
        self.ops, self.L, self.dev = ops, lmax, torch.device(device)
        L = lmax

        def it(x):
            return torch.tensor(np.asarray(x, dtype=np.int64), dtype=torch.int, device=self.dev)

        ltuples = [[] for _ in range(L + 1)]
        for l, l1, l2 in o.decode_triples(L, llls):
            ltuples[l].append((l1, l2))
        _, table = o.encode_sorted(ltuples)
        t_ff, t_off = o.tau_ff_and_offsets(L, taus, llls)
        self.taus, self.tau_out, self.t_ff = list(taus), list(tau_out), t_ff
        self.d_t_F, self.d_cum_F = it(taus), it(o.cumulative_tm(taus))
        self.d_t_FF, self.d_cum_FF = it(t_ff), it(o.cumulative_tm(t_ff))
        self.d_t_O, self.d_cum_O = it(tau_out), it(o.cumulative_tm(tau_out))
        self.d_cum_W = it(np.concatenate([[0], np.cumsum(t_ff * np.asarray(tau_out))]))
        self.d_llls, self.d_table = it(llls), it(table)
        self.d_t_off = it(list(t_off) + [2 ** 30])   # one spare entry: the kernel may peek one past the last triple
        offs = o.cg_offsets(L, llls)
        self.d_cg_off = it(offs)
        self.CG = torch.zeros(offs[-1], dtype=torch.float, device=self.dev)
        ops.sparse_precomputeCG(self.CG, L, self.d_llls, self.d_cg_off)
        self.n_F = int(o.cumulative_tm(taus)[-1])
        self.n_FF, self.n_O = int(o.cumulative_tm(t_ff)[-1]), int(o.cumulative_tm(tau_out)[-1])
        self.w_len, self.sum_tff = int((t_ff * np.asarray(tau_out)).sum()), int(t_ff.sum())

    @classmethod
    def from_case(cls, ops, case, device):
        return cls(ops, case["lmax"], case["taus"], case["tau_out"], case["llls"], device)

    def fits_int32(self, B):
        """The reference indexes its activations with 32-bit integers (`IDX`, cudaCG_sparse.cu:17)."""
        return 2 * B * max(self.n_FF, 1) < 2 ** 31

    def product_fwd(self, F):
        FF = torch.zeros(F.shape[0], self.n_FF, 2, device=self.dev)
        self.ops.sparse_forward(F, FF, self.L, F.shape[0], self.d_t_F, self.d_cum_F, self.d_t_FF, self.d_cum_FF, self.d_llls,
                                self.d_table, self.d_t_off, self.CG, self.d_cg_off)
        return FF

    def product_bwd(self, F, gFF):
        gF = torch.zeros_like(F)
        self.ops.sparse_backward(F, gF, gFF, self.L, F.shape[0], self.d_t_F, self.d_cum_F, self.d_t_FF, self.d_cum_FF, self.d_llls,
                                 self.d_t_off, self.CG, self.d_cg_off)
        return gF

    def _stds(self, stds, eps):
        return stds if stds is not None else torch.full((1,), eps, device=self.dev)

    def mix_fwd(self, FF, W, stds, cnt, eps, flags):
        O = torch.zeros(FF.shape[0], self.n_O, 2, device=self.dev)
        self.ops.FN_WMM_forward(FF, O, W, self.L, FF.shape[0], self.sum_tff, self.n_O, self.d_t_FF, self.d_cum_FF, self.d_cum_O,
                                self.d_cum_W, self._stds(stds, eps), cnt, eps, flags)
        return O

    def mix_bwd(self, gO, FF, W, stds, cnt, eps, flags):
        gFF, gW = torch.zeros_like(FF), torch.zeros_like(W)
        self.ops.FN_WMM_backward(gO, gFF, gW, FF, W, self.L, FF.shape[0], self.n_FF, self.w_len, self.d_t_FF, self.d_cum_FF,
                                 self.d_t_O, self.d_cum_O, self.d_cum_W, self._stds(stds, eps), cnt, eps, flags)
        return gFF, gW


class _RefCGBN(torch.autograd.Function):
    """One CG layer through the reference kernels, with the saved tensors of CG_layers.py:44-50,186-190 (the product
    stays in memory between forward and backward)."""

    @staticmethod
    def forward(ctx, F, W, layer, stds, cnt, eps, flags):
        F = F.contiguous()
        FF = layer.product_fwd(F)
        O = layer.mix_fwd(FF, W, stds, cnt, eps, flags)
        ctx.layer, ctx.cnt, ctx.eps, ctx.flags = layer, cnt, eps, flags
        ctx.save_for_backward(F, FF, W, None if stds is None else stds.detach().clone())
        return O

    @staticmethod
    def backward(ctx, gO):
        F, FF, W, stds = ctx.saved_tensors
        gFF, gW = ctx.layer.mix_bwd(gO.contiguous(), FF, W, stds, ctx.cnt, ctx.eps, ctx.flags)
        gF = ctx.layer.product_bwd(F, gFF) if ctx.needs_input_grad[0] else None
        return gF, gW, None, None, None, None, None


class RefNetwork(torch.nn.Module):
    """A stack of CG layers on the reference kernels with the skip-concatenated l = 0 invariants of
    CGNet/CGNet.py:52-69, for timing a whole training or inference step of the reference's CUDA path."""

    def __init__(self, lmax, layer_taus, llls, device, norm=True, seed=0):
        super().__init__()
        ops = load_ops()
        self.dev = torch.device(device)
        self.layers = [RefLayer(ops, lmax, layer_taus[i], layer_taus[i + 1], llls, device) for i in range(len(layer_taus) - 1)]
        self.layer_taus = layer_taus
        g = torch.Generator().manual_seed(seed)
        self.W = torch.nn.ParameterList([torch.nn.Parameter((0.05 * torch.rand(L.w_len, 2, generator=g)).to(self.dev)) for L in self.layers])
        self.stds = [(0.5 + torch.rand(L.sum_tff, generator=g)).to(self.dev) if norm else None for L in self.layers]
        self.cnt = 1.0
        self.output_length = 2 * sum(int(t[0]) for t in layer_taus)

    def fits_int32(self, B):
        return all(L.fits_int32(B) for L in self.layers)

    def forward(self, x):
        B = x.shape[0]
        emb = [x[:, : int(self.layer_taus[0][0]), :].reshape(B, -1)]
        fs = x
        for i, L in enumerate(self.layers):
            flags = 0 if self.stds[i] is None else (3 if self.training else 1)
            fs = _RefCGBN.apply(fs, self.W[i], L, self.stds[i], self.cnt, 1e-5, flags)
            emb.append(fs[:, : int(self.layer_taus[i + 1][0]), :].reshape(B, -1))
        if self.training:
            self.cnt += 1.0
        return torch.cat(emb, 1)
