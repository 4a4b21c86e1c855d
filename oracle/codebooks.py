"""Lattice codebooks of the reference, restated with integer arithmetic.

Follows (reference paths):
  quantizers/e8_lattice.py:54-81,124-128  -- E8 shell expansion, 65 536 rows
      truncated to 65 535 by ``remove_last``; rows inside a shell come out of
      ``torch.unique(dim=0)`` in ascending lexicographic order.
  quantizers/e8_d4.py:37-88               -- D4 points popped from a heap keyed
      by (squared norm, coordinate tuple), binned into four parity classes, the
      first 128 of each class kept.
  quantizers/e8_lattice.py:39 / e8_d4.py:84 -- table = raw / radius in fp32.

The reference grows shells by adding root vectors; the result is the complete
set of lattice points of each squared norm, so this file enumerates them
directly (coordinates doubled so that everything is an exact small integer).
"""
from __future__ import annotations

import functools
import itertools

import numpy as np

E8_ROWS = 65535          # table rows after ``remove_last``
E8_SHELLS = 7            # squared norms 0, 2, ..., 12


def _points_with_norm(coords: np.ndarray, dim: int, max_n4: int) -> np.ndarray:
    """All ``dim``-vectors over ``coords`` (doubled coordinates) whose doubled
    squared norm is <= max_n4.  Built one coordinate at a time with pruning."""
    sq = coords.astype(np.int64) ** 2
    pts = np.zeros((1, 0), dtype=np.int8)
    n4 = np.zeros(1, dtype=np.int64)
    for _ in range(dim):
        new_n4 = n4[:, None] + sq[None, :]
        keep = new_n4 <= max_n4
        ri, ci = np.nonzero(keep)
        pts = np.concatenate([pts[ri], coords[ci][:, None].astype(np.int8)], axis=1)
        n4 = new_n4[ri, ci]
    return pts


@functools.lru_cache(maxsize=None)
def _e8_raw_doubled() -> np.ndarray:
    """(65536, 8) int8: the doubled E8 points in the reference's row order."""
    max_n4 = 4 * 2 * (E8_SHELLS - 1)                    # doubled coords: |2v|^2 = 4|v|^2
    ints = _points_with_norm(np.arange(-6, 7, 2), 8, max_n4)     # integer coordinates
    halfs = _points_with_norm(np.arange(-7, 8, 2), 8, max_n4)    # half-integer coordinates
    allp = np.concatenate([ints, halfs], axis=0).astype(np.int64)
    # E8 in the even coordinate system: coordinate sum is an even integer,
    # i.e. the doubled coordinates sum to a multiple of 4.
    allp = allp[allp.sum(axis=1) % 4 == 0]
    n4 = (allp ** 2).sum(axis=1)
    shells = []
    for s in range(E8_SHELLS):
        sh = allp[n4 == 8 * s]
        order = np.lexsort(sh.T[::-1])                  # ascending, first coordinate major
        shells.append(sh[order])
    return np.concatenate(shells, axis=0)[:65536].astype(np.int8)


def e8_raw_points() -> np.ndarray:
    """(65535, 8) float32 E8 lattice points, before the radius division."""
    return (_e8_raw_doubled()[:E8_ROWS].astype(np.float32) * np.float32(0.5))


@functools.lru_cache(maxsize=None)
def _d4_raw_doubled() -> np.ndarray:
    """(4, 128, 4) int8 doubled D4 codes: classes even-full, even-half,
    odd-full, odd-half (e8_d4.py:61-71), each in (norm, tuple) order."""
    coords = np.arange(-6, 7)                           # doubled: integers and halves
    pts = _points_with_norm(coords, 4, 4 * 7).astype(np.int64)
    par = pts % 2
    pts = pts[(par == par[:, :1]).all(axis=1)]          # all integer or all half-integer
    rows = sorted((int((p * p).sum()), tuple(p.tolist())) for p in pts)
    classes = {(0, 0): [], (0, 1): [], (1, 0): [], (1, 1): []}
    for _, p in rows:
        half = p[0] % 2                                 # 1 -> half-integer vector
        odd = (sum(p) // 2) % 2                         # parity of the (integer) coordinate sum
        classes[(odd, half)].append(p)
    out = np.array([classes[(0, 0)][:128], classes[(0, 1)][:128],
                    classes[(1, 0)][:128], classes[(1, 1)][:128]], dtype=np.int8)
    return out


def d4_raw_codes() -> np.ndarray:
    """(4, 128, 4) float32 D4 codes, before the radius division."""
    return _d4_raw_doubled().astype(np.float32) * np.float32(0.5)


def e8_table(radius: float = 1.6) -> np.ndarray:
    """(65535, 8) float32 = raw / radius, the table ``dequant`` indexes."""
    return e8_raw_points() / np.float32(radius)


def d4_table(radius: float = 1.75) -> np.ndarray:
    """(4, 128, 4) float32 = raw / radius."""
    return d4_raw_codes() / np.float32(radius)
