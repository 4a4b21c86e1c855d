"""Codebooks of the two EPTQ vector quantizers: generation and ``dequant``.

Mirrors the parts of the reference quantizers that inference needs
(quantizers/e8_lattice.py:18-52,54-81,111-128 and
quantizers/e8_d4.py:20-107,237-255): the tables, ``set_radius``,
``remove_last`` and ``dequant``.  Nearest-neighbour encoding is an offline step
of the quantizer and is not part of this package.

The tables are generated with exact integer arithmetic on doubled coordinates
and match the reference's tables row for row: E8 shells of squared norm
0, 2, ..., 12 each in ascending lexicographic order, cut to 65 536 rows; D4
points ordered by (squared norm, coordinates) and binned into the classes
even-full, even-half, odd-full, odd-half, 128 each.
"""
from __future__ import annotations

from typing import Optional

import torch


def _enumerate(coords: torch.Tensor, dim: int, max_sq: int) -> torch.Tensor:
    """All ``dim``-tuples over ``coords`` (int64) with sum of squares <= max_sq."""
    pts = torch.zeros((1, 0), dtype=torch.int64)
    sq = torch.zeros(1, dtype=torch.int64)
    csq = coords * coords
    for _ in range(dim):
        cand = sq[:, None] + csq[None, :]
        ri, ci = torch.nonzero(cand <= max_sq, as_tuple=True)
        pts = torch.cat([pts[ri], coords[ci][:, None]], dim=1)
        sq = cand[ri, ci]
    return pts


def _lex_order(p: torch.Tensor, lead: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Row permutation sorting by ``lead`` (if given) then by the columns, ascending."""
    order = torch.arange(p.shape[0])
    for c in range(p.shape[1] - 1, -1, -1):
        order = order[torch.sort(p[order, c], stable=True).indices]
    if lead is not None:
        order = order[torch.sort(lead[order], stable=True).indices]
    return order


def e8_raw_points() -> torch.Tensor:
    """(65536, 8) fp32 E8 points (even coordinate system), reference row order."""
    both = torch.cat([_enumerate(torch.arange(-6, 7, 2), 8, 48),
                      _enumerate(torch.arange(-7, 8, 2), 8, 48)])
    both = both[both.sum(1) % 4 == 0]
    n4 = (both * both).sum(1)
    order = _lex_order(both, lead=n4)
    return (both[order][:65536].to(torch.float32) * 0.5).contiguous()


def d4_raw_codes() -> torch.Tensor:
    """(4, 128, 4) fp32 D4 codes, reference class and row order."""
    pts = _enumerate(torch.arange(-6, 7), 4, 28)
    par = pts % 2
    pts = pts[(par == par[:, :1]).all(1)]
    pts = pts[_lex_order(pts, lead=(pts * pts).sum(1))]
    half = pts[:, 0] % 2
    odd = torch.div(pts.sum(1), 2, rounding_mode="floor") % 2
    classes = [pts[(odd == o) & (half == hf)][:128] for o, hf in ((0, 0), (0, 1), (1, 0), (1, 1))]
    return (torch.stack(classes).to(torch.float32) * 0.5).contiguous()


class E8LatticeQuantizer:
    """E8 codebook: ``points`` (rows, 8) fp32 = raw lattice points / radius."""

    DEFAULT_RADIUS = 1.6

    def __init__(self, device: str = "cpu", codebook: Optional[torch.Tensor] = None,
                 radius: Optional[float] = None):
        if codebook is not None:
            self.points, self._raw_points, self._radius = codebook, None, self.DEFAULT_RADIUS
            return
        self._raw_points = e8_raw_points().to(device)
        self._radius = self.DEFAULT_RADIUS if radius is None else radius
        self.points = self._raw_points / self._radius

    def set_radius(self, new_radius: float) -> None:
        if self._raw_points is not None:
            self.points = self._raw_points / new_radius
        else:
            self.points = self.points * (self._radius / new_radius)
        self._radius = new_radius

    def remove_last(self) -> None:
        """Drop the last row so that index 65535 is free to mark critical blocks."""
        self.points = self.points[:-1]
        if self._raw_points is not None:
            self._raw_points = self._raw_points[:-1]

    def dequant(self, indices: torch.Tensor, scale=1.0) -> torch.Tensor:
        """(out//8, in) indices -> (out, in) fp32."""
        M, N = indices.shape
        return self.points[indices.long()].permute(0, 2, 1).reshape(M * 8, N) * scale


class E8D4Quantizer:
    """E8-D4 codebook: ``codes`` (4, 128, 4) fp32 = raw D4 codes / radius.  An index
    packs class (2 bits), i (7 bits), j (7 bits) and decodes to
    ``[codes[class, i], codes[class, j]]``."""

    DEFAULT_RADIUS = 1.875

    def __init__(self, device: str = "cpu", codebook: Optional[torch.Tensor] = None,
                 radius: Optional[float] = None):
        if codebook is not None:
            self.codes, self._raw_codes, self._radius = codebook, None, self.DEFAULT_RADIUS
            return
        self._raw_codes = d4_raw_codes().to(device)
        self._radius = self.DEFAULT_RADIUS if radius is None else radius
        self.codes = self._raw_codes / self._radius

    def set_radius(self, new_radius: float) -> None:
        if self._raw_codes is not None:
            self.codes = self._raw_codes / new_radius
        else:
            self.codes = self.codes * (self._radius / new_radius)
        self._radius = new_radius

    def remove_last(self) -> None:
        """Nothing to drop: 65535 = (3, 127, 127) is simply never emitted."""

    def dequant(self, indices: torch.Tensor, scale=1.0) -> torch.Tensor:
        idx = indices.long()
        ct, ii, jj = (idx >> 14) & 3, (idx >> 7) & 127, idx & 127
        vec = torch.cat([self.codes[ct, ii], self.codes[ct, jj]], dim=-1)   # (M, N, 8)
        M, N = idx.shape
        return vec.permute(0, 2, 1).reshape(M * 8, N) * scale
