"""Network-level composition of CG layers (reference: ``CGNet/CGNet.py:14-69``), plus the ``SphericalCNN_fast`` front
end whose source is absent from the reference repository and is reconstructed from its only call site
(``Shrec17/Shrec17_main_fast.py:78-92,136-147``)."""
import numpy as np
import torch
from torch import nn

from .cg_layers import CGBN_cuda

REAL_PART, IMAG_PART = 0, 1


class SphericalCNN(nn.Module):
    """A stack of ``CGBN_cuda`` layers; the invariant embedding is the concatenation of every layer's l=0 fragment
    (``skipconn=True``, including the input's) or the last layer's only.

    ``taus`` is a list of per-degree channel lists, ``taus[i]`` for the input of layer i, so ``len(taus)-1`` layers.
    Activations stay in the flat ``(B, N, 2)`` layout between layers (the reference converts to a list of views and
    back with ``torch.cat`` at every layer, ``CG_layers.py:275``); the result is identical.
    """

    def __init__(self, lmax, taus, cuda=True, norm=True, skipconn=True, sparse_flag=False, device="cuda", fused=True,
                 depthwise=False, init="random"):
        assert cuda, "Do not support these parameters yet"
        super().__init__()
        self.lmax = lmax
        self.taus = taus
        self.n_layers = len(taus) - 1
        self.cgs = nn.ModuleList([CGBN_cuda(lmax, taus[i], taus[i + 1], batchnorm=norm, sparse_flag=sparse_flag,
                                            device=device, fused=fused, depthwise=depthwise, init=init)
                                  for i in range(self.n_layers)])
        self.skipconn = skipconn
        if self.skipconn:
            self.output_length = 2 * sum(int(t[0]) for t in taus)
        else:
            self.output_length = 2 * int(taus[-1][0])
        self.to(device)

    def forward(self, f_input):
        if isinstance(f_input, (list, tuple)):
            B = f_input[0].shape[0]
            fs = torch.cat([v.reshape(B, -1, 2) for v in f_input], dim=1)
        else:
            B = f_input.shape[0]
            fs = f_input
        # the l=0 fragments are the first tau_0 rows of the flat activations: strided views, gathered by one concatenation
        embedding = [fs[:, : int(self.taus[0][0]), :]] if self.skipconn else []
        for i in range(self.n_layers):
            fs = self.cgs[i](fs, straight_output=True)
            if self.skipconn:
                embedding.append(fs[:, : int(self.taus[i + 1][0]), :])
        if self.skipconn:
            return torch.cat(embedding, 1).reshape(B, -1)
        return fs[:, : int(self.taus[-1][0]), :].reshape(B, -1)


class SphericalCNN_fast(SphericalCNN):
    """``SphericalCNN_fast(lmax, taus, nlayers, skip_type=1, num_channels_input=6)``.

    Takes spherical-harmonic coefficients of ``num_channels_input`` functions, complex, shape
    ``(B, C, (lmax+1)**2)`` with coefficient (l, m) at index ``l*l + l + m`` (numpy complex array, complex tensor, or a
    real tensor with a trailing (re, im) axis), rearranges them into fragments ``tau_l = C`` and runs ``nlayers`` CG
    layers with per-degree widths ``taus``.  ``skip_type`` 0 disables the skip concatenation, 1 enables it.
    """

    def __init__(self, lmax, taus, nlayers, skip_type=1, num_channels_input=1, norm=True, sparse_flag=False,
                 device="cuda", fused=True, depthwise=False):
        layer_taus = [[int(num_channels_input)] * (lmax + 1)] + [list(taus) for _ in range(nlayers)]
        super().__init__(lmax, layer_taus, cuda=True, norm=norm, skipconn=bool(skip_type), sparse_flag=sparse_flag,
                         device=device, fused=fused, depthwise=depthwise)
        self.num_channels_input = int(num_channels_input)
        idx = np.concatenate([c * (lmax + 1) ** 2 + np.arange(l * l, (l + 1) ** 2)
                              for l in range(lmax + 1) for c in range(self.num_channels_input)])
        self.register_buffer("_gather", torch.as_tensor(idx, dtype=torch.long, device=device), persistent=False)

    def pack(self, coeffs):
        """``(B, C, (lmax+1)^2)`` complex -> flat ``(B, sum_l C(2l+1), 2)`` float32 on the module's device."""
        if isinstance(coeffs, np.ndarray):
            coeffs = torch.from_numpy(coeffs)
        if coeffs.is_complex():
            coeffs = torch.view_as_real(coeffs.to(torch.complex64))
        coeffs = coeffs.to(device=self._gather.device, dtype=torch.float32)
        B = coeffs.shape[0]
        return coeffs.reshape(B, -1, 2).index_select(1, self._gather)

    def forward(self, coeffs):
        return super().forward(self.pack(coeffs))
