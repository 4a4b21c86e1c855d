"""Readers of the on-disk layout the reference's quantizer writes
(quantize.py:36-127,425-437; README.md:131-152):

    <dir>/quant_config.json            quantisation settings (only `quantizer_type` matters here)
    <dir>/quantizer.pt                 {quantizer_type, raw_codes, radius, warp_alpha} or legacy {codebook[, saved_radius]}
    <dir>/config.json                  HuggingFace model config
    <dir>/non_quantized_params.pt      embeddings, final norm, lm_head
    <dir>/layer_<i>/<linear name>.pt   QuantizedLayerData dictionaries
    <dir>/layer_<i>/non_quantized.pt   layer norms

Same function names as the reference's loaders (reconstruct.py:32-108)."""
from __future__ import annotations

import json
from pathlib import Path
from typing import Dict, Tuple

import torch

from .config import QuantizedLayerData


def load_quantization_config(quantized_dir: Path) -> Dict:
    with open(Path(quantized_dir) / "quant_config.json") as f:
        return json.load(f)


def load_codebook(quantized_dir: Path) -> Tuple[torch.Tensor, torch.Tensor, float, str]:
    """(codebook fp32 already divided by the radius, raw codes or None, radius, quantizer_type).

    New format: codebook = raw_codes / radius, exactly as reconstruct.py:51-62 rebuilds it.  A radially
    warped codebook (warp_alpha != 1, quantizers/e8_d4.py:282-298) is reproduced as well; the reference's
    kernel loader ignores it (kernels/patch.py:52-58)."""
    data = torch.load(Path(quantized_dir) / "quantizer.pt", weights_only=True, map_location="cpu")
    qtype = data.get("quantizer_type", "e8_lattice")
    if "raw_codes" in data:
        raw = data["raw_codes"].float()
        radius = float(data["radius"])
        cb = raw / radius
        alpha = float(data.get("warp_alpha", 1.0))
        if alpha != 1.0 and qtype == "e8_d4":
            flat = cb.reshape(-1, 4)
            norms = flat.norm(dim=1)
            max_norm = norms.max()
            new_norms = (norms / max_norm.clamp(min=1e-8)).pow(alpha) * max_norm
            scale = torch.where(norms > 1e-8, new_norms / norms, torch.zeros_like(norms))
            cb = (flat * scale.unsqueeze(1)).reshape(4, 128, 4)
            raw = None                      # per-layer radii cannot be re-derived from warped codes
        return cb.contiguous(), raw, radius, qtype
    radius = float(data.get("saved_radius", 0.0)) or float(load_quantization_config(quantized_dir).get("codebook_radius") or 0.0)
    return data["codebook"].float().contiguous(), None, radius, qtype


def load_quantized_layer(layer_dir: Path, layer_name: str) -> QuantizedLayerData:
    return QuantizedLayerData.load(Path(layer_dir) / f"{layer_name}.pt")


def load_global_non_quantized_params(quantized_dir: Path) -> Dict[str, torch.Tensor]:
    return torch.load(Path(quantized_dir) / "non_quantized_params.pt", weights_only=True, map_location="cpu")


def load_layer_non_quantized_params(layer_dir: Path) -> Dict[str, torch.Tensor]:
    return torch.load(Path(layer_dir) / "non_quantized.pt", weights_only=True, map_location="cpu")
