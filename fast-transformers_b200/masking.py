"""Mask objects handed to attention layers (1 / True = keep).

Mirror of the classes of ``fast_transformers/masking.py`` that the causal-linear path
reads: ``BaseMask`` derived views (:23-114), ``FullMask`` (:117-161), ``LengthMask``
(:164-192) and ``TriangularCausalMask`` (:195-206).  ``CausalLinearAttention`` only asks
``attn_mask.lower_triangular`` and ``key_lengths.float_matrix`` / ``.lengths``.
"""
import torch


class BaseMask(object):
    @property
    def bool_matrix(self):
        raise NotImplementedError()

    @property
    def float_matrix(self):
        if not hasattr(self, "_float_matrix"):
            with torch.no_grad():
                self._float_matrix = self.bool_matrix.float()
        return self._float_matrix

    @property
    def lengths(self):
        """Number of leading ones per row; ValueError if a row is not ones-then-zeros."""
        if not hasattr(self, "_lengths"):
            with torch.no_grad():
                m = self.bool_matrix
                lengths = m.long().sum(dim=-1)
                cols = torch.arange(m.shape[-1], device=m.device)
                expected = cols.view(*([1] * (m.dim() - 1)), -1) < lengths.unsqueeze(-1)
                if not torch.equal(expected, m):
                    raise ValueError("The mask is not a length mask")
                self._lengths = lengths
        return self._lengths

    @property
    def shape(self):
        return self.bool_matrix.shape

    @property
    def additive_matrix(self):
        if not hasattr(self, "_additive_matrix"):
            with torch.no_grad():
                self._additive_matrix = torch.log(self.bool_matrix.float())
        return self._additive_matrix

    @property
    def additive_matrix_finite(self):
        if not hasattr(self, "_additive_matrix_finite"):
            with torch.no_grad():
                self._additive_matrix_finite = (~self.bool_matrix).float() * (-1e24)
        return self._additive_matrix_finite

    @property
    def all_ones(self):
        if not hasattr(self, "_all_ones"):
            with torch.no_grad():
                self._all_ones = torch.all(self.bool_matrix)
        return self._all_ones

    @property
    def lower_triangular(self):
        """True when row i keeps exactly the first i+1 entries."""
        if not hasattr(self, "_lower_triangular"):
            self._lower_triangular = False
            with torch.no_grad():
                try:
                    lengths = self.lengths
                    if lengths.dim() == 1:
                        target = torch.arange(1, len(lengths) + 1, device=lengths.device)
                        self._lower_triangular = bool(torch.all(lengths == target))
                except ValueError:
                    pass
        return self._lower_triangular


class FullMask(BaseMask):
    """Wraps a bool tensor, or builds an all-True N x M mask (``FullMask(N)``,
    ``FullMask(N, M)`` or keyword forms)."""

    def __init__(self, mask=None, N=None, M=None, device="cpu"):
        if mask is not None and isinstance(mask, torch.Tensor):
            if mask.dtype != torch.bool:
                raise ValueError("FullMask expects the mask to be bool")
            with torch.no_grad():
                self._mask = mask.clone()
            return
        if mask is not None and M is None and isinstance(mask, int):
            M = N
            N = mask
        if N is not None:
            M = M or N
            with torch.no_grad():
                self._mask = torch.ones(N, M, dtype=torch.bool, device=device)
            self._all_ones = True
            return
        raise ValueError("Either mask or N should be provided")

    @property
    def bool_matrix(self):
        return self._mask


class LengthMask(BaseMask):
    """Rows of ones up to ``lengths[i]``; ``max_len`` defaults to ``lengths.max()``."""

    def __init__(self, lengths, max_len=None, device=None):
        self._device = device or lengths.device
        with torch.no_grad():
            self._lengths = lengths.clone().to(self._device)
        self._max_len = max_len or self._lengths.max()
        self._bool_matrix = None
        self._all_ones = torch.all(self._lengths == self._max_len).item()

    @property
    def bool_matrix(self):
        if self._bool_matrix is None:
            with torch.no_grad():
                idx = torch.arange(self._max_len, device=self._device)
                self._bool_matrix = idx.view(1, -1) < self._lengths.view(-1, 1)
        return self._bool_matrix


class TriangularCausalMask(LengthMask):
    """N x N lower-triangular mask (diagonal kept)."""

    def __init__(self, N, device="cpu"):
        super().__init__(torch.arange(1, N + 1, device=device), N, device)
        self._lower_triangular = True
