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


def write_quantized_dir(path, hf_config, quantizer, quantizer_type: str, seed: int = 42, outlier_frac: float = 0.002,
                        dtype=torch.float16, init_std: float = 0.02):
    """Write a random-init model in the layout the reference's quantizer produces (quantize.py:36-127):
    config.json, quant_config.json, quantizer.pt, non_quantized_params.pt, layer_<i>/<linear>.pt and
    layer_<i>/non_quantized.pt.  Linears are synthetic layers (make_layer); norms are ones, embeddings
    and lm_head are N(0, init_std).  Returns {(layer index, linear name): QuantizedLayerData}."""
    import json
    from pathlib import Path

    from transformers import AutoModelForCausalLM

    from .kernels.patch import _parameters_on_meta, decoder_layers, linear_layers

    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    hf_config.save_pretrained(path)
    (path / "quant_config.json").write_text(json.dumps({"quantizer_type": quantizer_type, "model_name": ""}))
    raw = quantizer._raw_points if quantizer_type == "e8_lattice" else quantizer._raw_codes
    torch.save({"quantizer_type": quantizer_type, "raw_codes": raw.float().cpu(), "radius": quantizer._radius,
                "warp_alpha": 1.0}, path / "quantizer.pt")
    with _parameters_on_meta():
        model = AutoModelForCausalLM.from_config(hf_config, dtype=dtype)
    gen = torch.Generator().manual_seed(seed)
    layers = decoder_layers(model)
    out = {}
    layer_param_names = set()
    for lid, layer in enumerate(layers):
        ldir = path / f"layer_{lid}"
        ldir.mkdir(exist_ok=True)
        for k, (name, lin) in enumerate(linear_layers(layer).items()):
            qd = make_layer(lin.out_features, lin.in_features, seed=seed + 1000 * lid + k, outlier_frac=outlier_frac,
                            bias=lin.bias is not None, scale_sigma=0.05)
            qd.g = (qd.g.float() * (init_std * 1.5)).to(torch.float16)        # keep activations O(1) through the stack
            qd.save(ldir / f"{name}.pt")
            out[(lid, name)] = qd
        norms = {}
        for name, module in layer.named_modules():
            if "norm" in name.lower():
                for pn, p in module.named_parameters(recurse=False):
                    full = f"{name}.{pn}" if name else pn
                    norms[full] = torch.zeros(p.shape, dtype=dtype) if pn == "bias" else torch.ones(p.shape, dtype=dtype)
        torch.save(norms, ldir / "non_quantized.pt")
    layer_ids = {id(p) for layer in layers for p in layer.parameters()}
    glob = {}
    for name, p in model.named_parameters():
        if id(p) in layer_ids:
            continue
        if "norm" in name.lower():
            glob[name] = torch.zeros(p.shape, dtype=dtype) if name.endswith("bias") else torch.ones(p.shape, dtype=dtype)
        else:
            glob[name] = (torch.randn(p.shape, generator=gen) * init_std).to(dtype)
    torch.save(glob, path / "non_quantized_params.pt")
    return out
