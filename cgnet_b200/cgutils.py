"""Host-side index layer of the Clebsch-Gordan layer: which (l1, l2) pairs feed each output degree, their canonical
order, and the offsets that give every mid channel and every weight column its meaning.

Same names, arguments and results as the reference's ``CGNet/CGutils.py`` for everything on the CUDA path
(``SparseLtuples``, ``compute_MST``, ``reshape_out``, ``calc_prod_taus``, ``Complex_bmm``); the CPU-only pieces of that
file (the dense Clebsch-Gordan dictionary for the pure-Python layer) have no counterpart here.
"""
import numpy as np
import torch

REAL_PART, IMAG_PART = 0, 1


def Complex_bmm(w, f):
    """Batched complex matmul on split (…, 2) tensors, ``w @ f`` (reference: ``CGutils.py:15-21``)."""
    wc = torch.view_as_complex(w.contiguous())
    fc = torch.view_as_complex(f.contiguous())
    return torch.view_as_real(torch.bmm(wc, fc))


def calc_prod_taus(lmax, taus, taus2=None):
    """Mid-channel count per degree for the full pair list (reference: ``CGutils.py:33-41``)."""
    taus2 = taus if taus2 is None else taus2
    assert len(taus) == len(taus2) == lmax + 1
    out = [0] * (lmax + 1)
    for l1 in range(lmax + 1):
        for l2 in range(l1 + 1):
            for l in range(l1 - l2, min(l1 + l2, lmax) + 1):
                out[l] += taus[l1] * taus2[l2]
    return out


def compute_MST(l, lmax, diag=False):
    """Pairs on a minimum spanning tree over the degrees 0..lmax for output degree ``l``
    (reference: ``CGutils.py:73-98``).

    An edge joins a < b whenever (a, b, l) is admissible, weight (2l+1)(2a+1)(2b+1).  Returns ``(l1s, l2s)`` with
    ``l1 > l2`` for tree edges, followed (``diag=True``) by every (a, a) with ``l <= 2a``.  The tree among
    equal-weight alternatives is whatever scipy's ``minimum_spanning_tree`` picks for the matrix built exactly the
    way the reference builds it (edge stored at row b, column a), so both agree for a given scipy version.
    """
    from scipy.sparse import csr_matrix
    from scipy.sparse.csgraph import minimum_spanning_tree

    a, b = np.triu_indices(lmax + 1, k=1)                    # a < b, in the reference's (row-major) edge order
    ok = (b - a <= l) & (l <= a + b)
    a, b = a[ok], b[ok]
    weights = (2 * l + 1) * (2 * a + 1) * (2 * b + 1)
    tree = minimum_spanning_tree(csr_matrix((weights, (b, a)), shape=(lmax + 1, lmax + 1))).tocoo()
    l1s, l2s = tree.row.tolist(), tree.col.tolist()
    if diag:
        extra = [d for d in range(lmax + 1) if l <= 2 * d]
        l1s += extra
        l2s += extra
    return l1s, l2s


class SparseLtuples:
    """Pair lists and their flattened representation (reference: ``CGutils.py:101-187``)."""

    @classmethod
    def compute_default_ltuples(cls, lmax):
        """All ``l2 <= l1 <= lmax`` with ``l1-l2 <= l <= min(l1+l2, lmax)``, enumerated l1-major."""
        out = [[] for _ in range(lmax + 1)]
        for l1 in range(lmax + 1):
            for l2 in range(l1 + 1):
                for l in range(l1 - l2, min(l1 + l2, lmax) + 1):
                    out[l].append((l1, l2))
        return out

    @classmethod
    def compute_debug_ltuples(cls, lmax):
        """The first two pairs of the default list for every degree."""
        return [pairs[:2] for pairs in cls.compute_default_ltuples(lmax)]

    @classmethod
    def compute_mst_ltuples(cls, lmax):
        """Per-degree MST pair lists with the diagonal added (what the reference's ``lll_mode='mst'`` expands to,
        ``CG_layers.py:226-230``)."""
        return [list(zip(*compute_MST(l, lmax, diag=True))) for l in range(lmax + 1)]

    @classmethod
    def sparse_rep_ltuples_sorted(cls, ltuples):
        """Encode the pairs of every degree, stably sorted by l1, as ``(l(L+1)+l1)(L+1)+l2`` and build the flattened
        ``(L+1) x (L+2)`` table whose entry (l, l1) is the index of the first triple of degree l whose first operand is
        >= l1 (entry (l, L+1) = one past the last triple of degree l)."""
        lmax = len(ltuples) - 1
        L1 = lmax + 1
        codes = []
        table = np.zeros((L1, L1 + 1), dtype=np.int64)
        for l in range(L1):
            pairs = np.asarray(ltuples[l], dtype=np.int64).reshape(-1, 2)
            assert (pairs[:, 0] >= pairs[:, 1]).all(), "pairs must satisfy l1 >= l2"
            order = np.argsort(pairs[:, 0], kind="stable")
            pairs = pairs[order]
            table[l, 0] = len(codes)
            table[l, 1:] = len(codes) + np.cumsum(np.bincount(pairs[:, 0], minlength=L1))
            codes += ((l * L1 + pairs[:, 0]) * L1 + pairs[:, 1]).tolist()
        return codes, table.reshape(-1)

    @classmethod
    def get_iter(cls, lmax, llls):
        """Decode to a list of ``(l, l1, l2)``."""
        c = np.asarray(llls, dtype=np.int64)
        L1 = lmax + 1
        return list(zip((c // (L1 * L1)).tolist(), ((c // L1) % L1).tolist(), (c % L1).tolist()))

    @classmethod
    def cal_CG_offsets(cls, lmax, llls):
        """Start of each triple's ``(2l+1) x (2l2+1)`` band in the CG table, with the total length appended."""
        c = np.asarray(llls, dtype=np.int64)
        L1 = lmax + 1
        sizes = (2 * (c // (L1 * L1)) + 1) * (2 * (c % L1) + 1)
        return np.concatenate([[0], np.cumsum(sizes)]).astype(np.int64).tolist()

    @classmethod
    def get_CG_length(cls, lmax, llls):
        return cls.cal_CG_offsets(lmax, llls)[-1]

    @classmethod
    def cal_new_tau_and_offsets(cls, lmax, taus, llls, depthwise=False):
        """Mid channels per degree and the first mid channel of every triple (reference: ``CG_layers.py:253-262``).
        ``depthwise`` counts tau_l1 channels per triple instead of tau_l1*tau_l2 (an extension, not in the reference)."""
        t_FF = np.zeros(lmax + 1, dtype=int)
        offsets = []
        for l, l1, l2 in cls.get_iter(lmax, llls):
            offsets.append(int(t_FF[l]))
            t_FF[l] += taus[l1] if depthwise else taus[l1] * taus[l2]
        return t_FF, offsets


def cumulative_tm(taus):
    """``[0, tau_0*1, tau_0*1 + tau_1*3, ...]``: start of every fragment in the flat activation."""
    taus = np.asarray(taus, dtype=np.int64)
    return np.concatenate([[0], np.cumsum(taus * (2 * np.arange(len(taus)) + 1))])


def reshape_out(output, taus):
    """Flat ``(B, N, 2)`` -> list of ``(B, tau_l, 2l+1, 2)`` views (reference: ``CGutils.py:190-197``)."""
    ret, offset = [], 0
    for l, t in enumerate(taus):
        t = int(t)
        ret.append(output[:, offset: offset + (2 * l + 1) * t, :].view(-1, t, 2 * l + 1, 2))
        offset += (2 * l + 1) * t
    assert offset == output.shape[1]
    return ret
