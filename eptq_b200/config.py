"""On-disk / in-memory format of one quantized linear layer.

Mirror of the reference's ``QuantizedLayerData`` (config.py:98-159): same field
names, same ``torch.save`` dictionary keys, ``load`` always lands on the CPU.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Any, Dict, Optional

import torch

_REQUIRED = ("Q", "g", "h", "O")
_OPTIONAL = ("bias", "chosen_r", "S_group")


@dataclass
class QuantizedLayerData:
    """Q: int16 (out//8, in) = codebook index - 32768, 32767 marks a critical block.
    g: (out,) row scales.  h: (in,) column scales.  O: (n_marked, 8) values of the
    critical blocks in row-major marker order.  bias: (out,) or None.
    chosen_r: codebook radius this layer was quantized with, or None.
    S_group: (out//qb_size, in) group scales, or None."""

    Q: torch.Tensor
    g: torch.Tensor
    h: torch.Tensor
    O: torch.Tensor
    bias: Optional[torch.Tensor] = None
    chosen_r: Optional[float] = None
    S_group: Optional[torch.Tensor] = None

    def to_dict(self) -> Dict[str, Any]:
        out = {k: getattr(self, k) for k in _REQUIRED}
        for k in _OPTIONAL:
            v = getattr(self, k)
            if v is not None:
                out[k] = v
        return out

    @classmethod
    def from_dict(cls, d: Dict[str, Any]) -> "QuantizedLayerData":
        return cls(**{k: d[k] for k in _REQUIRED}, **{k: d.get(k) for k in _OPTIONAL})

    def save(self, path: Path) -> None:
        torch.save(self.to_dict(), path)

    @classmethod
    def load(cls, path: Path) -> "QuantizedLayerData":
        return cls.from_dict(torch.load(path, weights_only=True, map_location="cpu"))

    @property
    def out_features(self) -> int:
        return int(self.Q.shape[0]) * 8

    @property
    def in_features(self) -> int:
        return int(self.Q.shape[1])
