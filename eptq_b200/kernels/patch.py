"""load_quantized_model: build a HuggingFace causal LM whose decoder linears are EPTQLinear modules.

Same signature and behaviour as the reference (kernels/patch.py:24-142): the model skeleton is created
without allocating weights, every ``nn.Linear`` inside a decoder layer is replaced by an ``EPTQLinear``
built from ``layer_<i>/<name>.pt``, norms / embeddings / lm_head come from the non-quantized files, the
codebook is one shared tensor.  Differences: no dependency on ``accelerate``; a layer quantized at its
own radius (``chosen_r``) gets the table of that radius, as the reference's reconstruction does
(algorithms/eptq.py:432-434) and its kernel loader does not; ``require_tokenizer=False`` lets a
directory without tokenizer files load (returns ``None`` for it)."""
from __future__ import annotations

import contextlib
import sys
from pathlib import Path
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from ..loaders import (load_codebook, load_global_non_quantized_params, load_layer_non_quantized_params,
                       load_quantization_config, load_quantized_layer)
from .linear import EPTQLinear


@contextlib.contextmanager
def _parameters_on_meta():
    """Create modules with their parameters on the meta device (buffers stay real), like
    accelerate.init_empty_weights which the reference uses (kernels/patch.py:65)."""
    original = nn.Module.register_parameter

    def register(module, name, param):
        original(module, name, param)
        if param is not None:
            cls = type(module._parameters[name])
            module._parameters[name] = cls(module._parameters[name].to("meta"), requires_grad=False)

    nn.Module.register_parameter = register
    try:
        yield
    finally:
        nn.Module.register_parameter = original


def decoder_layers(model: nn.Module) -> nn.ModuleList:
    """Decoder layer list of an OPT or LLaMA-style model (models/opt.py:14-16, models/llama.py:14-16)."""
    name = model.__class__.__name__.lower()
    if "opt" in name:
        return model.model.decoder.layers
    if "llama" in name or hasattr(getattr(model, "model", None), "layers"):
        return model.model.layers
    raise ValueError(f"Unsupported model type: {model.__class__.__name__}")


def linear_layers(layer: nn.Module) -> Dict[str, nn.Linear]:
    """Every nn.Linear of a decoder layer by dotted name (models/llama.py:62-68)."""
    return {n: m for n, m in layer.named_modules() if isinstance(m, nn.Linear)}


def _set_by_path(root: nn.Module, dotted: str, value) -> None:
    parts = dotted.split(".")
    target = root
    for part in parts[:-1]:
        target = getattr(target, part)
    setattr(target, parts[-1], value)


def load_quantized_model(quantized_dir: str, device: str = "cuda", require_tokenizer: bool = True,
                         tp_rank: int = 0, tp_size: int = 1) -> Tuple[nn.Module, Optional[object]]:
    """(model, tokenizer) with quantized decoder linears.  ``tp_size > 1`` keeps this rank's shard of
    every linear (see eptq_b200.parallel); the caller owns the all-reduce after row-parallel layers."""
    from transformers import AutoConfig, AutoModelForCausalLM

    quantized_dir = Path(quantized_dir)
    quant_config = load_quantization_config(quantized_dir)
    quantizer_type = quant_config.get("quantizer_type", "e8_lattice")

    print("Loading codebook...", file=sys.stderr)
    codebook, raw_codes, radius, _ = load_codebook(quantized_dir)
    codebook = codebook.to(device)
    per_radius: Dict[float, torch.Tensor] = {}

    print("Creating model structure...", file=sys.stderr)
    config = AutoConfig.from_pretrained(quantized_dir)
    dtype = getattr(config, "dtype", None) or getattr(config, "torch_dtype", None) or torch.float16
    if isinstance(dtype, str):
        dtype = getattr(torch, dtype)
    with _parameters_on_meta():
        model = AutoModelForCausalLM.from_config(config, dtype=dtype)

    tokenizer = None
    try:
        from transformers import AutoTokenizer
        tokenizer = AutoTokenizer.from_pretrained(quantized_dir / "tokenizer")
    except Exception:
        model_name = quant_config.get("model_name")
        if require_tokenizer:
            if not model_name:
                raise ValueError("Tokenizer not found in quantized_dir/tokenizer and "
                                 "'model_name' missing from quant_config.json.")
            from transformers import AutoTokenizer
            tokenizer = AutoTokenizer.from_pretrained(model_name)

    layers = decoder_layers(model)
    print(f"Loading {len(layers)} quantized layers...", file=sys.stderr)
    if tp_size > 1:
        from ..parallel import shard_layer
    for lid, layer in enumerate(layers):
        layer_dir = quantized_dir / f"layer_{lid}"
        for name in linear_layers(layer):
            qd = load_quantized_layer(layer_dir, name)
            if tp_size > 1:
                qd = shard_layer(qd, name, tp_rank, tp_size)
            cb = codebook
            if qd.chosen_r is not None and raw_codes is not None and float(qd.chosen_r) != radius:
                r = float(qd.chosen_r)
                if r not in per_radius:
                    per_radius[r] = (raw_codes / r).to(device)
                cb = per_radius[r]
            _set_by_path(layer, name, EPTQLinear.from_quantized_data(qd, cb, quantizer_type))
        for pname, param in load_layer_non_quantized_params(layer_dir).items():
            _set_by_path(layer, pname, nn.Parameter(param, requires_grad=False))

    for pname, param in load_global_non_quantized_params(quantized_dir).items():
        _set_by_path(model, pname, nn.Parameter(param, requires_grad=False))

    missing = [n for n, p in model.named_parameters() if p.is_meta]
    if missing:
        print(f"WARNING: {len(missing)} meta parameters not loaded: {missing[:5]}", file=sys.stderr)

    model = model.to(device=device)
    model.eval()
    print("Quantized model loaded.", file=sys.stderr)
    return model, tokenizer
