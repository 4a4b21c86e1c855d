"""load_quantized_model on a synthetic directory in the reference's on-disk layout (CPU part: structure;
GPU part: logits against an fp16 model rebuilt from the oracle's reconstructed weights)."""
import numpy as np
import pytest
import torch
import torch.nn as nn

import oracle
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.kernels.patch import load_quantized_model
from eptq_b200.loaders import load_codebook, load_quantized_layer
from eptq_b200.quantizers import E8D4Quantizer, E8LatticeQuantizer
from eptq_b200.synthetic import write_quantized_dir
from tests import util


def llama_config():
    from transformers import LlamaConfig
    return LlamaConfig(hidden_size=128, intermediate_size=352, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=2, vocab_size=512, max_position_embeddings=256,
                       tie_word_embeddings=False)


def opt_config():
    from transformers import OPTConfig
    return OPTConfig(hidden_size=96, ffn_dim=384, num_hidden_layers=2, num_attention_heads=4, vocab_size=512,
                     max_position_embeddings=128, word_embed_proj_dim=96)


def test_directory_layout_and_structure(tmp_path):
    qds = write_quantized_dir(tmp_path, llama_config(), E8D4Quantizer(radius=1.75), "e8_d4")
    for f in ("config.json", "quant_config.json", "quantizer.pt", "non_quantized_params.pt",
              "layer_0/self_attn.q_proj.pt", "layer_1/mlp.down_proj.pt", "layer_1/non_quantized.pt"):
        assert (tmp_path / f).exists(), f
    cb, raw, radius, qtype = load_codebook(tmp_path)
    assert qtype == "e8_d4" and radius == 1.75 and np.array_equal(cb.numpy(), oracle.d4_table(1.75))
    back = load_quantized_layer(tmp_path / "layer_0", "mlp.up_proj")
    assert torch.equal(back.Q, qds[(0, "mlp.up_proj")].Q)

    model, tok = load_quantized_model(str(tmp_path), device="cpu", require_tokenizer=False)
    assert tok is None
    names = {n for n, m in model.named_modules() if isinstance(m, EPTQLinear)}
    assert len(names) == 14 and "model.layers.1.mlp.gate_proj" in names
    assert not any(isinstance(m, nn.Linear) for layer in model.model.layers for m in layer.modules())
    assert isinstance(model.lm_head, nn.Linear)                       # not quantized (quantize.py:86-90)
    assert not any(p.is_meta for p in model.parameters())
    lins = [m for m in model.modules() if isinstance(m, EPTQLinear)]
    assert all(m._codebook is lins[0]._codebook for m in lins)       # one shared table
    with pytest.raises(ValueError):
        load_quantized_model(str(tmp_path), device="cpu")             # no tokenizer and no model_name


def test_per_layer_radius_and_tensor_parallel_shards(tmp_path):
    qds = write_quantized_dir(tmp_path, llama_config(), E8D4Quantizer(radius=1.75), "e8_d4")
    qd = qds[(0, "mlp.up_proj")]
    qd.chosen_r = 1.9
    qd.save(tmp_path / "layer_0" / "mlp.up_proj.pt")
    model, _ = load_quantized_model(str(tmp_path), device="cpu", require_tokenizer=False)
    up, gate = model.model.layers[0].mlp.up_proj, model.model.layers[0].mlp.gate_proj
    assert np.array_equal(up._codebook32.numpy().reshape(4, 128, 4), oracle.d4_table(1.9))
    assert np.array_equal(gate._codebook32.numpy().reshape(4, 128, 4), oracle.d4_table(1.75))
    m1, _ = load_quantized_model(str(tmp_path), device="cpu", require_tokenizer=False, tp_rank=1, tp_size=2)
    assert m1.model.layers[0].mlp.up_proj.out_features == 176 and m1.model.layers[0].mlp.up_proj.in_features == 128
    assert m1.model.layers[0].mlp.down_proj.in_features == 176 and m1.model.layers[0].mlp.down_proj.out_features == 128


def _reference_model(path, cfg, qds, table, kind):
    """fp16 HuggingFace model with the oracle's reconstructed weights (the reference's reconstruct path)."""
    from transformers import AutoModelForCausalLM
    from eptq_b200.kernels.patch import decoder_layers, linear_layers
    model = AutoModelForCausalLM.from_config(cfg, dtype=torch.float16)
    sd = torch.load(path / "non_quantized_params.pt")
    model.load_state_dict(sd, strict=False)
    for lid, layer in enumerate(decoder_layers(model)):
        for name, lin in linear_layers(layer).items():
            qd = qds[(lid, name)]
            lin.weight.data = torch.from_numpy(oracle.dequantize_layer(util.qld_arrays(qd), table))
            if qd.bias is not None:
                lin.bias.data = qd.bias.clone()
        layer.load_state_dict(torch.load(path / f"layer_{lid}" / "non_quantized.pt"), strict=False)
    return model.eval()


@pytest.mark.gpu
@pytest.mark.parametrize("arch,kind", [("llama", "e8_d4"), ("opt", "e8_lattice"), ("llama", "e8_lattice")])
def test_logits_match_reconstructed_model(tmp_path, arch, kind):
    from eptq_b200.decode import decode
    cfg = llama_config() if arch == "llama" else opt_config()
    if kind == "e8_d4":
        quantizer, table = E8D4Quantizer(radius=1.75), oracle.d4_table(1.75)
    else:
        quantizer = E8LatticeQuantizer(radius=1.6)
        quantizer.remove_last()
        table = oracle.e8_table(1.6)
    qds = write_quantized_dir(tmp_path, cfg, quantizer, kind, outlier_frac=0.01)
    model, _ = load_quantized_model(str(tmp_path), device="cuda", require_tokenizer=False)
    ref = _reference_model(tmp_path, cfg, qds, table, kind).to("cuda")
    ids = torch.randint(0, 512, (2, 24), generator=torch.Generator().manual_seed(3)).to("cuda")
    with torch.no_grad():
        a = model(input_ids=ids).logits.float()
        b = ref(input_ids=ids).logits.float()
    assert float((a - b).abs().max() / b.abs().max()) < 6e-2           # two fp16 models, 2 layers deep, small logits
    toks, stats = decode(model, ids[:1], max_new_tokens=6)
    ref_toks, _ = decode(ref, ids[:1], max_new_tokens=6)
    assert toks.shape == (1, 6) and stats["tokens_per_s"] > 0
    assert (toks == ref_toks).float().mean() >= 0.5                    # greedy paths agree except at near-ties
