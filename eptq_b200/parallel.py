"""Tensor-parallel sharding of quantized layers (one process per GPU).

The reference is single-device (kernels/patch.py:24-27,138); this module adds
Megatron-style sharding on top of its format without changing the format:

* column-parallel (q/k/v/gate/up, OPT q/k/v/fc1): rank r keeps the Q rows
  ``[r*M/T, (r+1)*M/T)`` with their ``g``, ``bias`` and ``S_group`` rows; because
  ``O`` is stored in row-major marker order (algorithms/eptq.py:376-378) its
  share is one contiguous slice.  ``h`` is replicated.  Outputs stay sharded.
* row-parallel (o/down, OPT out_proj/fc2): rank r keeps the Q columns
  ``[r*N/T, (r+1)*N/T)`` with their ``h`` and ``S_group`` columns and the rows of
  ``O`` whose marker column falls in the range (order kept).  ``g`` is
  replicated and applied before the reduction (scaling is linear); the bias is
  kept on rank 0 only.  Outputs are partial sums: all-reduce them.
"""
from __future__ import annotations

from typing import Optional

import torch

from .config import QuantizedLayerData

COLUMN_PARALLEL = {"q_proj", "k_proj", "v_proj", "gate_proj", "up_proj", "fc1"}
ROW_PARALLEL = {"o_proj", "down_proj", "out_proj", "fc2"}
MARKER = 32767


def parallel_kind(name: str) -> Optional[str]:
    leaf = name.split(".")[-1]
    if leaf in COLUMN_PARALLEL:
        return "column"
    if leaf in ROW_PARALLEL:
        return "row"
    return None


def shard_columnwise(qd: QuantizedLayerData, rank: int, world: int) -> QuantizedLayerData:
    """Output-row shard (column-parallel linear)."""
    M = qd.Q.shape[0]
    out_f = M * 8
    if M % world:
        raise ValueError(f"out_features/8 = {M} does not divide over {world} ranks")
    m0, m1 = rank * M // world, (rank + 1) * M // world
    S = qd.S_group
    if S is not None:
        qb = out_f // S.shape[0]
        if (8 * m0) % qb or (8 * m1) % qb:
            raise ValueError("shard boundary splits a scale group")
        S = S[8 * m0 // qb: 8 * m1 // qb].contiguous()
    marks = (qd.Q == MARKER)
    before = int(marks[:m0].sum().item())
    inside = int(marks[m0:m1].sum().item())
    return QuantizedLayerData(
        Q=qd.Q[m0:m1].contiguous(), g=qd.g[8 * m0: 8 * m1].contiguous(), h=qd.h,
        O=qd.O[before: before + inside].contiguous(),
        bias=None if qd.bias is None else qd.bias[8 * m0: 8 * m1].contiguous(),
        chosen_r=qd.chosen_r, S_group=S)


def shard_rowwise(qd: QuantizedLayerData, rank: int, world: int, align: int = 8) -> QuantizedLayerData:
    """Input-column shard (row-parallel linear); partial outputs must be summed over ranks."""
    N = qd.Q.shape[1]
    if N % (world * align):
        raise ValueError(f"in_features = {N} does not divide into {world} shards of a multiple of {align}")
    n0, n1 = rank * N // world, (rank + 1) * N // world
    rows, cols = (qd.Q == MARKER).nonzero(as_tuple=True)
    keep = (cols >= n0) & (cols < n1)
    bias = qd.bias if rank == 0 else None
    return QuantizedLayerData(
        Q=qd.Q[:, n0:n1].contiguous(), g=qd.g, h=qd.h[n0:n1].contiguous(),
        O=qd.O[keep].contiguous(), bias=bias, chosen_r=qd.chosen_r,
        S_group=None if qd.S_group is None else qd.S_group[:, n0:n1].contiguous())


def shard_layer(qd: QuantizedLayerData, name: str, rank: int, world: int) -> QuantizedLayerData:
    """Shard by the layer's name; layers that are neither kind are replicated."""
    if world == 1:
        return qd
    kind = parallel_kind(name)
    if kind == "column":
        return shard_columnwise(qd, rank, world)
    if kind == "row":
        return shard_rowwise(qd, rank, world)
    return qd


def shard_activation(x: torch.Tensor, rank: int, world: int) -> torch.Tensor:
    """Slice of the last dimension a row-parallel layer of this rank consumes."""
    n = x.shape[-1]
    return x[..., rank * n // world: (rank + 1) * n // world]
