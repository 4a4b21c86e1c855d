"""Token-by-token decode loop over a model returned by ``load_quantized_model``: prefill once, then
one forward per new token with the key/value cache, greedy or top-k sampling.  Timing follows the
reference's protocol (bench_decode.py:44-71): the prefill is excluded, tokens/s = (new tokens - 1) /
time of the per-token loop."""
from __future__ import annotations

import time
from typing import Dict, Tuple

import torch


@torch.no_grad()
def decode(model, input_ids: torch.Tensor, max_new_tokens: int, top_k: int = 0,
           temperature: float = 1.0) -> Tuple[torch.Tensor, Dict[str, float]]:
    """Returns (generated ids (batch, max_new_tokens), {"prefill_s", "decode_s", "tokens_per_s"})."""
    device = input_ids.device
    if device.type == "cuda":
        # cuDNN attention re-plans for every new key length (about 10 ms per call on B200 with this
        # PyTorch), which would swamp a per-token loop; the flash / memory-efficient kernels do not.
        torch.backends.cuda.enable_cudnn_sdp(False)
    sync = torch.cuda.synchronize if device.type == "cuda" else (lambda: None)
    sync()
    t0 = time.perf_counter()
    out = model(input_ids=input_ids, use_cache=True)
    past = out.past_key_values
    nxt = _pick(out.logits[:, -1], top_k, temperature)
    sync()
    t1 = time.perf_counter()
    tokens = [nxt]
    for _ in range(max_new_tokens - 1):
        out = model(input_ids=nxt[:, None], past_key_values=past, use_cache=True)
        past = out.past_key_values
        nxt = _pick(out.logits[:, -1], top_k, temperature)
        tokens.append(nxt)
    sync()
    t2 = time.perf_counter()
    n = max(max_new_tokens - 1, 1) * input_ids.shape[0]
    return torch.stack(tokens, dim=1), {"prefill_s": t1 - t0, "decode_s": t2 - t1, "tokens_per_s": n / max(t2 - t1, 1e-9)}


def _pick(logits: torch.Tensor, top_k: int, temperature: float) -> torch.Tensor:
    if top_k <= 0:
        return logits.argmax(dim=-1)
    vals, idx = torch.topk(logits.float() / max(temperature, 1e-6), top_k, dim=-1)
    choice = torch.multinomial(torch.softmax(vals, dim=-1), 1)
    return idx.gather(-1, choice).squeeze(-1)


def _main():
    """Whole-model decode on a random-init model of a named architecture, written to a temporary
    directory in the quantizer's on-disk layout and loaded with load_quantized_model."""
    import argparse
    import json
    import tempfile

    from transformers import LlamaConfig

    from .kernels.patch import load_quantized_model
    from .quantizers import E8D4Quantizer, E8LatticeQuantizer
    from .synthetic import write_quantized_dir

    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="llama2-7b", choices=["llama2-7b", "tiny"])
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--quantizer", default="e8_d4", choices=["e8_d4", "e8_lattice"])
    ap.add_argument("--prefill", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    args = ap.parse_args()
    if args.arch == "llama2-7b":
        cfg = LlamaConfig(hidden_size=4096, intermediate_size=11008, num_hidden_layers=args.layers or 32,
                          num_attention_heads=32, num_key_value_heads=32, vocab_size=32000,
                          max_position_embeddings=4096, tie_word_embeddings=False)
    else:
        cfg = LlamaConfig(hidden_size=256, intermediate_size=704, num_hidden_layers=args.layers or 2,
                          num_attention_heads=8, num_key_value_heads=8, vocab_size=1024,
                          max_position_embeddings=2048, tie_word_embeddings=False)
    if args.quantizer == "e8_d4":
        q = E8D4Quantizer(radius=1.75)
    else:
        q = E8LatticeQuantizer(radius=1.6)
        q.remove_last()
    with tempfile.TemporaryDirectory() as d:
        t0 = time.perf_counter()
        write_quantized_dir(d, cfg, q, args.quantizer)
        t1 = time.perf_counter()
        model, _ = load_quantized_model(d, device="cuda", require_tokenizer=False)
        t2 = time.perf_counter()
    ids = torch.randint(0, cfg.vocab_size, (args.batch, args.prefill), generator=torch.Generator().manual_seed(0)).cuda()
    decode(model, ids[:, :8], 4)                                   # warm-up
    _, stats = decode(model, ids, args.new_tokens)
    print(json.dumps({"arch": args.arch, "layers": cfg.num_hidden_layers, "quantizer": args.quantizer,
                      "batch": args.batch, "prefill_tokens": args.prefill, "new_tokens": args.new_tokens,
                      "write_dir_s": t1 - t0, "load_s": t2 - t1, **stats,
                      "note": "eager HuggingFace forward, one kernel launch per linear, no CUDA graph"}))


if __name__ == "__main__":
    _main()
