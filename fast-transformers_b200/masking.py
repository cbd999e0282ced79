"""Keep-masks (True / 1 = attend) handed to the attention layers of this package.

Only what the linear-attention path asks of a mask is implemented: the causal layer reads
``attn_mask.lower_triangular`` and ``key_lengths.float_matrix`` / ``.lengths``
(``fast_transformers/attention/causal_linear_attention.py:80-83``), the non-causal layer reads
``attn_mask.all_ones`` (``fast_transformers/attention/linear_attention.py:63-66``), the
encoder builds default masks (``fast_transformers/transformers.py:129-132``).  The
constructors keep the reference's names and argument order (``fast_transformers/masking.py``:
``FullMask`` :117, ``LengthMask`` :164, ``TriangularCausalMask`` :195), so the reference's own
mask objects and these are interchangeable for the layers here; additive (log) forms, which
only the softmax attentions use, are left out.

One class does the work: a mask is stored either as per-row prefix lengths (no matrix is
built until somebody asks for one) or as a dense bool matrix.
"""
import torch


class Mask(object):
    """A 2-D keep-mask, ``rows x width``.

    ``prefix``: int64 tensor (rows,), row r keeps its first ``prefix[r]`` entries; or
    ``dense``: bool tensor (rows, width)."""

    def __init__(self, prefix=None, width=None, dense=None):
        self._prefix, self._width, self._dense = prefix, width, dense
        self._float = None
        self._flags = {}

    # ---- views --------------------------------------------------------------------------
    @property
    def bool_matrix(self):
        if self._dense is None:
            cols = torch.arange(int(self._width), device=self._prefix.device)
            self._dense = cols[None, :] < self._prefix[:, None]
        return self._dense

    @property
    def float_matrix(self):
        if self._float is None:
            self._float = self.bool_matrix.to(torch.float32)
        return self._float

    @property
    def shape(self):
        if self._dense is not None:
            return self._dense.shape
        return torch.Size((self._prefix.shape[0], int(self._width)))

    @property
    def lengths(self):
        """Entries kept per row, for a mask whose rows are ones followed by zeros;
        ``ValueError`` for any other mask."""
        if self._prefix is None:
            m = self._dense
            # a row is a prefix exactly when no kept entry follows a dropped one
            if m.shape[-1] > 1 and bool((m[..., 1:] & ~m[..., :-1]).any()):
                raise ValueError("The mask is not a length mask")
            self._prefix = m.sum(dim=-1, dtype=torch.int64)
        return self._prefix

    # ---- predicates ---------------------------------------------------------------------
    @property
    def all_ones(self):
        if "ones" not in self._flags:
            if self._dense is not None:
                self._flags["ones"] = bool(self._dense.all())
            else:
                self._flags["ones"] = bool((self._prefix >= int(self._width)).all())
        return self._flags["ones"]

    @property
    def lower_triangular(self):
        """Square-or-wider mask whose row i keeps exactly entries 0..i."""
        if "tril" not in self._flags:
            try:
                n = self.lengths
                want = torch.arange(1, n.shape[0] + 1, device=n.device)
                self._flags["tril"] = n.dim() == 1 and bool(torch.equal(n, want))
            except ValueError:
                self._flags["tril"] = False
        return self._flags["tril"]


class FullMask(Mask):
    """``FullMask(bool_tensor)`` wraps a dense mask; ``FullMask(N)``, ``FullMask(N, M)`` (also
    by keyword) is an all-True mask of that size."""

    def __init__(self, mask=None, N=None, M=None, device="cpu"):
        if isinstance(mask, torch.Tensor):
            if mask.dtype != torch.bool:
                raise ValueError("FullMask expects the mask to be bool")
            super().__init__(dense=mask.detach().clone())
            return
        if isinstance(mask, int) and M is None:
            N, M = mask, N
        if N is None:
            raise ValueError("Either mask or N should be provided")
        M = M or N
        super().__init__(prefix=torch.full((N,), M, dtype=torch.int64, device=device), width=M)


class LengthMask(Mask):
    """Row r keeps its first ``lengths[r]`` entries; ``max_len`` defaults to the longest row."""

    def __init__(self, lengths, max_len=None, device=None):
        n = lengths.detach().to(device=device or lengths.device, dtype=torch.int64).clone()
        super().__init__(prefix=n, width=int(max_len) if max_len else int(n.max()))


class TriangularCausalMask(LengthMask):
    """``N x N`` causal mask: position i attends to positions 0..i."""

    def __init__(self, N, device="cpu"):
        super().__init__(torch.arange(1, N + 1, device=device), max_len=N)
        self._flags["tril"] = True
