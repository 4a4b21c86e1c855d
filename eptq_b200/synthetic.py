"""Seeded synthetic ``QuantizedLayerData`` with the value distributions of the
benchmark configurations: indices uniform over the valid codebook range
(0..65534), a Bernoulli fraction of critical-block markers with N(0,1) fp16
values, log-normal fp16 row/column scales, optional log-normal group scales.
These stand in for real quantized checkpoints, which need the model hub."""
from __future__ import annotations

from typing import Optional

import torch

from .config import QuantizedLayerData

LLAMA2_7B_LINEARS = {      # name -> (out_features, in_features)
    "self_attn.q_proj": (4096, 4096), "self_attn.k_proj": (4096, 4096),
    "self_attn.v_proj": (4096, 4096), "self_attn.o_proj": (4096, 4096),
    "mlp.gate_proj": (11008, 4096), "mlp.up_proj": (11008, 4096), "mlp.down_proj": (4096, 11008),
}
LLAMA3_8B_LINEARS = {
    "self_attn.q_proj": (4096, 4096), "self_attn.k_proj": (1024, 4096),
    "self_attn.v_proj": (1024, 4096), "self_attn.o_proj": (4096, 4096),
    "mlp.gate_proj": (14336, 4096), "mlp.up_proj": (14336, 4096), "mlp.down_proj": (4096, 14336),
}


def make_layer(out_features: int, in_features: int, seed: int = 42, outlier_frac: float = 0.002,
               bias: bool = False, qb_size: Optional[int] = None, device: str = "cpu",
               scale_sigma: float = 0.25) -> QuantizedLayerData:
    """One synthetic layer.  The random stream depends on (seed, device type) only."""
    dev = torch.device(device)
    gen = torch.Generator(device=dev)
    gen.manual_seed(seed)
    M, N = out_features // 8, in_features
    idx = torch.randint(0, 65535, (M, N), generator=gen, device=dev, dtype=torch.int32)
    marked = torch.rand((M, N), generator=gen, device=dev) < outlier_frac
    idx = torch.where(marked, torch.full_like(idx, 65535), idx)
    Q = (idx - 32768).to(torch.int16)
    n_marked = int(marked.sum().item())
    O = torch.randn((n_marked, 8), generator=gen, device=dev).to(torch.float16)
    g = torch.exp(scale_sigma * torch.randn(out_features, generator=gen, device=dev)).to(torch.float16)
    h = torch.exp(scale_sigma * torch.randn(in_features, generator=gen, device=dev)).to(torch.float16)
    b = torch.randn(out_features, generator=gen, device=dev).to(torch.float16) if bias else None
    S = None
    if qb_size:
        S = torch.exp(0.1 * torch.randn((out_features // qb_size, in_features), generator=gen, device=dev))
        S = S.to(torch.float16)
    return QuantizedLayerData(Q=Q, g=g, h=h, O=O, bias=b, S_group=S)


def make_activations(batch: int, in_features: int, seed: int = 43, device: str = "cpu") -> torch.Tensor:
    gen = torch.Generator(device=torch.device(device))
    gen.manual_seed(seed)
    return torch.randn((batch, in_features), generator=gen, device=device).to(torch.float16)
