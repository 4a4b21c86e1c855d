"""Reconstruction and layer-output oracle, restated in numpy.

Follows (reference paths):
  algorithms/eptq.py:406-471   ``dequantize_layer``: index -> table row (fp32),
      optional group scale, critical blocks patched from ``O`` in row-major
      marker order, then ``* g[:,None] * h[None,:]`` left to right in fp32 and
      one round to fp16.
  quantizers/e8_lattice.py:111-122 and quantizers/e8_d4.py:237-255  ``dequant``.
  kernels/linear.py:122-139    CSR side tables built from ``Q == 32767``.
  test_e8_cuda.py:23-53        second, independent statement of the GEMV
      formula (table lookup, h*x in fp32, CSR correction, row scale).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import numpy as np

MARKER_I16 = 32767           # stored value of index 65535 (algorithms/eptq.py:389-393)


@dataclass
class LayerArrays:
    """numpy view of the reference's ``QuantizedLayerData`` (config.py:98-159)."""
    Q: np.ndarray                       # int16 (out//8, in)
    g: np.ndarray                       # fp16 (out,)
    h: np.ndarray                       # fp16 (in,)
    O: np.ndarray                       # fp16 (n_masked, 8)
    bias: Optional[np.ndarray] = None   # fp16 (out,)
    S_group: Optional[np.ndarray] = None  # fp16 (out//qb, in)


def _lookup(Q_idx: np.ndarray, table: np.ndarray) -> np.ndarray:
    """(M, N) int32 indices -> (M, 8, N) float32 codewords."""
    if table.ndim == 3:                                 # E8-D4 (4,128,4): e8_d4.py:248-255
        ct = (Q_idx >> 14) & 3
        ii = (Q_idx >> 7) & 0x7F
        jj = Q_idx & 0x7F
        a1 = table[ct, ii]                              # (M, N, 4)
        a2 = table[ct, jj]
        vec = np.concatenate([a1, a2], axis=-1)         # (M, N, 8)
    else:                                               # E8 (rows, 8): e8_lattice.py:122
        vec = table[Q_idx]
    return np.ascontiguousarray(vec.transpose(0, 2, 1))


def dequantize_layer(layer: LayerArrays, table: np.ndarray) -> np.ndarray:
    """fp16 (out, in) weight, bit-for-bit what the reference reconstructs.

    ``table`` is the fp32 codebook already divided by the radius that applies
    to this layer (the reference swaps the radius in for ``chosen_r`` and back,
    algorithms/eptq.py:432-434,456-457)."""
    table = np.asarray(table, dtype=np.float32)
    Q_idx = layer.Q.astype(np.int32) + 32768
    mask = Q_idx == 65535
    Q_idx = np.where(mask, 0, Q_idx)
    M, N = Q_idx.shape
    W = _lookup(Q_idx, table)                           # (M, 8, N) fp32
    if layer.S_group is not None:
        S = layer.S_group.astype(np.float32)            # (out//qb, in)
        qb = (M * 8) // S.shape[0]
        W = W.reshape(M * 8, N) * np.repeat(S, qb, axis=0)
        W = W.reshape(M, 8, N)
    if layer.O.size:
        r, c = np.nonzero(mask)                         # row-major order
        W[r, :, c] = layer.O.astype(np.float32)
    W = W.reshape(M * 8, N)
    W = (W * layer.g.astype(np.float32)[:, None]) * layer.h.astype(np.float32)[None, :]
    return W.astype(np.float16)


def linear_reference(x: np.ndarray, W16: np.ndarray,
                     bias: Optional[np.ndarray] = None) -> np.ndarray:
    """fp32 (B, out): x.float() @ W16.float().T (+ bias)."""
    y = x.astype(np.float32) @ W16.astype(np.float32).T
    if bias is not None:
        y = y + bias.astype(np.float32)[None, :]
    return y


def csr_from_q(Q: np.ndarray):
    """(O_col int32 (n,), O_row_ptr int32 (M+1,)) as linear.py:122-139 builds them."""
    r, c = np.nonzero(Q == MARKER_I16)
    counts = np.bincount(r, minlength=Q.shape[0])
    ptr = np.concatenate([[0], np.cumsum(counts)]).astype(np.int32)
    return c.astype(np.int32), ptr


def gemv_formula_reference(layer: LayerArrays, table16: np.ndarray, x: np.ndarray) -> np.ndarray:
    """fp32 (B, out) from the un-reconstructed formula the reference's kernels
    evaluate: y = g * (sum_unmarked cb[q]*h*x + sum_marked O*h*x) + bias, with an
    fp16 table (test_e8_cuda.py:23-53).  Group scales are not part of it."""
    assert layer.S_group is None
    tab = np.asarray(table16, dtype=np.float16).astype(np.float32)
    Q_idx = layer.Q.astype(np.int32) + 32768
    mask = Q_idx == 65535
    Wc = _lookup(np.where(mask, 0, Q_idx), tab)         # (M, 8, N)
    Wc = Wc * (~mask)[:, None, :]
    xh = x.astype(np.float32) * layer.h.astype(np.float32)[None, :]
    y = np.einsum("mkn,bn->bmk", Wc, xh)
    col, ptr = csr_from_q(layer.Q)
    Of = layer.O.astype(np.float32)
    for m in range(Q_idx.shape[0]):
        for i in range(ptr[m], ptr[m + 1]):
            y[:, m, :] += Of[i][None, :] * xh[:, col[i]][:, None]
    y = y.reshape(x.shape[0], -1) * layer.g.astype(np.float32)[None, :]
    if layer.bias is not None:
        y = y + layer.bias.astype(np.float32)[None, :]
    return y
