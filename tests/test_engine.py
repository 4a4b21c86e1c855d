"""Decode engine against the HuggingFace forward of the same weights: on the CPU with dense fp32
linears (checks norm, rotary embedding, cache and mask logic), on the GPU with quantized layers
(checks the grouped launches and the captured CUDA graph)."""
import tempfile

import pytest
import torch

from eptq_b200.engine import LlamaDecodeEngine


def _tiny_config(kv_heads=4):
    from transformers import LlamaConfig
    return LlamaConfig(hidden_size=64, intermediate_size=160, num_hidden_layers=2, num_attention_heads=4,
                       num_key_value_heads=kv_heads, vocab_size=128, max_position_embeddings=64,
                       tie_word_embeddings=False)


@pytest.mark.parametrize("kv_heads", [4, 2])
def test_engine_matches_hf_forward_cpu(kv_heads):
    from transformers import LlamaForCausalLM
    torch.manual_seed(0)
    model = LlamaForCausalLM(_tiny_config(kv_heads)).float().eval()
    eng = LlamaDecodeEngine.from_model(model, max_len=32, batch=2)
    ids = torch.randint(0, 128, (2, 9))
    with torch.no_grad():
        ref = model(input_ids=ids).logits
        got = eng.forward_reference(ids[:, :6], torch.arange(6))
        assert torch.allclose(got, ref[:, :6], atol=2e-4, rtol=1e-3)
        for p in range(6, 9):                       # token by token over the cache
            step = eng.forward_reference(ids[:, p:p + 1], torch.tensor([p]))
            assert torch.allclose(step[:, 0], ref[:, p], atol=2e-4, rtol=1e-3)


def test_engine_greedy_state_cpu():
    from transformers import LlamaForCausalLM
    torch.manual_seed(1)
    model = LlamaForCausalLM(_tiny_config()).float().eval()
    eng = LlamaDecodeEngine.from_model(model, max_len=32, batch=1)
    ids = torch.randint(0, 128, (1, 5))
    with torch.no_grad():
        first = eng.prefill(ids)
        seq = [int(first)]
        for _ in range(3):
            eng._step()
            seq.append(int(eng.next_token))
        full = torch.cat([ids, torch.tensor([seq[:-1]])], dim=1)
        ref = model(input_ids=full).logits[0, 4:].argmax(-1).tolist()
    assert seq == ref
    assert int(eng.position) == 8


@pytest.mark.gpu
@pytest.mark.parametrize("quantizer_type,hidden,heads,inter", [("e8_d4", 256, 8, 704), ("e8_lattice", 256, 8, 704),
                                                              ("e8_d4", 512, 4, 768), ("e8_lattice", 512, 4, 768)])
def test_engine_graph_decode_gpu(quantizer_type, hidden, heads, inter):
    from eptq_b200.kernels.patch import load_quantized_model
    from eptq_b200.quantizers import E8D4Quantizer, E8LatticeQuantizer
    from eptq_b200.synthetic import write_quantized_dir
    from transformers import LlamaConfig

    cfg = LlamaConfig(hidden_size=hidden, intermediate_size=inter, num_hidden_layers=2, num_attention_heads=heads,
                      num_key_value_heads=heads, vocab_size=512, max_position_embeddings=256, tie_word_embeddings=False)
    if quantizer_type == "e8_d4":
        q = E8D4Quantizer(radius=1.75)
    else:
        q = E8LatticeQuantizer(radius=1.6)
        q.remove_last()
    with tempfile.TemporaryDirectory() as d:
        write_quantized_dir(d, cfg, q, quantizer_type)
        model, _ = load_quantized_model(d, device="cuda", require_tokenizer=False)
    ids = torch.randint(0, 512, (1, 24), generator=torch.Generator().manual_seed(3)).cuda()
    eng = LlamaDecodeEngine.from_model(model, max_len=64, batch=1)
    plain = LlamaDecodeEngine.from_model(model, max_len=64, batch=1)
    pos = torch.arange(24, device="cuda")
    with torch.no_grad():
        ref = model(input_ids=ids).logits.float()
        got = eng.forward(ids, pos).float()                       # fused kernels, prompt-sized
        same = plain.forward_reference(ids, pos).float()          # plain PyTorch statement
        scale = float(ref.abs().max())
        assert float((got - ref).abs().max()) <= 2e-2 * scale
        assert float((same - ref).abs().max()) <= 2e-2 * scale
        # one more token through the single-query attention kernel against the plain statement
        nxt = ids[:, :1]
        p1 = torch.tensor([24], device="cuda")
        a = eng.forward(nxt, p1).float()
        b = plain.forward_reference(nxt, p1).float()
        assert float((a - b).abs().max()) <= 2e-2 * scale
        # head size 128 takes the fully fused step (norm, rotary, cache, residual in the GEMVs)
        assert (eng._fused not in (None, False)) == (hidden // heads == 128)
        if eng._fused and eng._chainable():
            # the same token with a layer's four GEMV stages as ONE chained launch instead of four launches
            one = LlamaDecodeEngine.from_model(model, max_len=64, batch=1)
            one.one_launch_per_layer = True
            one.forward(ids, pos)
            c = one.forward(nxt, p1).float()
            assert float((c - b).abs().max()) <= 2e-2 * scale
    eager, _ = eng.decode(ids, 12, use_graph=False)
    graphed, stats = eng.decode(ids, 12, use_graph=True)
    assert eng.graph is not None
    assert torch.equal(eager, graphed)
    again, _ = eng.decode(ids, 12, use_graph=True)
    assert torch.equal(again, graphed)
    assert stats["tokens_per_s"] > 0


def _tp_engine_worker(rank, world, port, out):
    """Rank `rank` of a tensor-parallel engine on the CPU: dense fp32 shards of one tiny model (output rows of
    q/k/v/gate/up, input columns of o/down), gloo all-reduce, the plain PyTorch statement of the step."""
    import os

    import torch.distributed as dist
    import torch.nn as nn
    from transformers import LlamaForCausalLM

    from eptq_b200.engine import DecoderLayerWeights

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.manual_seed(0)
    model = LlamaForCausalLM(_tiny_config(4)).float().eval()

    def rows(lin):
        n = lin.out_features // world
        m = nn.Linear(lin.in_features, n, bias=False)
        m.weight.data = lin.weight.data[rank * n:(rank + 1) * n].clone()
        return m

    def cols(lin):
        n = lin.in_features // world
        m = nn.Linear(n, lin.out_features, bias=False)
        m.weight.data = lin.weight.data[:, rank * n:(rank + 1) * n].clone()
        return m
    core, cfg = model.model, model.config
    layers = [DecoderLayerWeights(rows(l.self_attn.q_proj), rows(l.self_attn.k_proj), rows(l.self_attn.v_proj),
                                  cols(l.self_attn.o_proj), rows(l.mlp.gate_proj), rows(l.mlp.up_proj),
                                  cols(l.mlp.down_proj), l.input_layernorm.weight.data,
                                  l.post_attention_layernorm.weight.data) for l in core.layers]
    hd = cfg.hidden_size // cfg.num_attention_heads
    eng = LlamaDecodeEngine(layers, core.embed_tokens.weight.data, core.norm.weight.data, model.lm_head.weight.data,
                            core.rotary_emb.inv_freq, cfg.rms_norm_eps, hd, cfg.num_attention_heads // world,
                            cfg.num_key_value_heads // world, max_len=32, batch=1, tp_group=dist.group.WORLD)
    ids = torch.randint(0, 128, (1, 7), generator=torch.Generator().manual_seed(5))
    with torch.no_grad():
        first = eng.prefill(ids)
        seq = [int(first)]
        for _ in range(3):
            eng._step()
            seq.append(int(eng.next_token))
        if rank == 0:
            full = torch.cat([ids, torch.tensor([seq[:-1]])], dim=1)
            ref = model(input_ids=full).logits[0, 6:].argmax(-1).tolist()
            torch.save({"seq": seq, "ref": ref}, out)
    dist.barrier()
    dist.destroy_process_group()


def test_engine_tensor_parallel_two_rank_gloo(tmp_path):
    """Heads split over two ranks, partial sums of o / down all-reduced: same greedy tokens as the whole model."""
    import os

    import torch.multiprocessing as mp
    out = str(tmp_path / "tp.pt")
    mp.spawn(_tp_engine_worker, args=(2, 29800 + os.getpid() % 1500, out), nprocs=2, join=True)
    got = torch.load(out)
    assert got["seq"] == got["ref"]


# ---- OPT (configuration 1's model family) -------------------------------------------------------------
def _tiny_opt_config():
    from transformers import OPTConfig
    return OPTConfig(hidden_size=64, ffn_dim=160, num_hidden_layers=2, num_attention_heads=4, vocab_size=128,
                     max_position_embeddings=64, word_embed_proj_dim=64, do_layer_norm_before=True,
                     dropout=0.0, attention_dropout=0.0)


def test_opt_engine_matches_hf_forward_cpu():
    from transformers import OPTForCausalLM
    from eptq_b200.engine import OPTDecodeEngine, decode_engine_for
    torch.manual_seed(0)
    model = OPTForCausalLM(_tiny_opt_config()).float().eval()
    eng = decode_engine_for(model, max_len=32, batch=2)
    assert isinstance(eng, OPTDecodeEngine)
    ids = torch.randint(0, 128, (2, 9))
    with torch.no_grad():
        ref = model(input_ids=ids).logits
        got = eng.forward_reference(ids[:, :6], torch.arange(6))
        assert torch.allclose(got, ref[:, :6], atol=2e-4, rtol=1e-3)
        for p in range(6, 9):                       # token by token over the cache
            step = eng.forward_reference(ids[:, p:p + 1], torch.tensor([p]))
            assert torch.allclose(step[:, 0], ref[:, p], atol=2e-4, rtol=1e-3)
        # greedy state machine
        eng2 = decode_engine_for(model, max_len=32, batch=1)
        first = eng2.prefill(ids[:1, :5])
        seq = [int(first)]
        for _ in range(3):
            eng2._step()
            seq.append(int(eng2.next_token))
        full = torch.cat([ids[:1, :5], torch.tensor([seq[:-1]])], dim=1)
        assert seq == model(input_ids=full).logits[0, 4:].argmax(-1).tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("quantizer_type", ["e8_lattice", "e8_d4"])
def test_opt_engine_graph_decode_gpu(quantizer_type):
    """OPT-125m-shaped layers (768 wide, heads of 64) with the E8 codebook of configuration 1: the engine's
    kernels against the HuggingFace forward over the same quantized modules, then graph replay against eager."""
    from eptq_b200.engine import OPTDecodeEngine, decode_engine_for
    from eptq_b200.kernels.patch import load_quantized_model
    from eptq_b200.quantizers import E8D4Quantizer, E8LatticeQuantizer
    from eptq_b200.synthetic import write_quantized_dir
    from transformers import OPTConfig

    cfg = OPTConfig(hidden_size=768, ffn_dim=3072, num_hidden_layers=2, num_attention_heads=12, vocab_size=512,
                    max_position_embeddings=256, word_embed_proj_dim=768, do_layer_norm_before=True,
                    dropout=0.0, attention_dropout=0.0)
    if quantizer_type == "e8_d4":
        q = E8D4Quantizer(radius=1.75)
    else:
        q = E8LatticeQuantizer(radius=1.6)
        q.remove_last()
    with tempfile.TemporaryDirectory() as d:
        write_quantized_dir(d, cfg, q, quantizer_type)
        model, _ = load_quantized_model(d, device="cuda", require_tokenizer=False)
    ids = torch.randint(0, 512, (1, 24), generator=torch.Generator().manual_seed(3)).cuda()
    eng = decode_engine_for(model, max_len=64, batch=1)
    assert isinstance(eng, OPTDecodeEngine)
    pos = torch.arange(24, device="cuda")
    with torch.no_grad():
        ref = model(input_ids=ids).logits.float()
        got = eng.forward(ids, pos).float()
        scale = float(ref.abs().max())
        assert float((got - ref).abs().max()) <= 2e-2 * scale
        nxt, p1 = ids[:, :1], torch.tensor([24], device="cuda")
        a = eng.forward(nxt, p1).float()                          # single-query attention kernel, heads of 64
        b = decode_engine_for(model, max_len=64, batch=1)
        b.forward_reference(ids, pos)
        assert float((a - b.forward_reference(nxt, p1).float()).abs().max()) <= 2e-2 * scale
    eager, _ = eng.decode(ids, 12, use_graph=False)
    graphed, stats = eng.decode(ids, 12, use_graph=True)
    assert torch.equal(eager, graphed)
    assert stats["tokens_per_s"] > 0
