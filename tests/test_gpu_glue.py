"""Decode-step glue kernels against their plain PyTorch statements (through the C ABI)."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _rot_half(x):
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


@pytest.mark.parametrize("rows,H", [(1, 4096), (3, 256), (512, 4096), (2, 8192 + 64)])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_rmsnorm(rows, H, with_delta):
    from eptq_b200.kernels import glue
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + H)
    x = torch.randn(rows, H, generator=g, device="cuda").half()
    d = torch.randn(rows, H, generator=g, device="cuda").half() if with_delta else None
    w = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).half()
    x_ref = x + d if with_delta else x.clone()
    xf = x_ref.float()
    n = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half()
    ref = w * n
    x_run = x.clone()
    out = glue.add_rmsnorm(x_run, w, 1e-5, d)
    assert torch.equal(x_run, x_ref)
    assert float((out.float() - ref.float()).abs().max()) <= 4e-3 * float(ref.float().abs().max())


def test_silu_mul():
    from eptq_b200.kernels import glue
    g = torch.Generator(device="cuda").manual_seed(5)
    a = (3 * torch.randn(2, 11008, generator=g, device="cuda")).half()
    b = torch.randn(2, 11008, generator=g, device="cuda").half()
    out = glue.silu_mul(a, b)
    ref = F.silu(a.float()) * b.float()
    assert float((out.float() - ref).abs().max()) <= 2e-3 * float(ref.abs().max())


@pytest.mark.parametrize("B,T,nh,nkv,hd", [(1, 1, 32, 32, 128), (2, 3, 8, 2, 64), (1, 17, 4, 4, 128)])
def test_rope_append(B, T, nh, nkv, hd):
    from eptq_b200.kernels import glue
    max_len = 96
    g = torch.Generator(device="cuda").manual_seed(B * 100 + T)
    q = torch.randn(B * T, nh * hd, generator=g, device="cuda").half()
    k = torch.randn(B * T, nkv * hd, generator=g, device="cuda").half()
    v = torch.randn(B * T, nkv * hd, generator=g, device="cuda").half()
    kc = torch.zeros(B, nkv, max_len, hd, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    pos = torch.arange(40, 40 + T, device="cuda")
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))
    ang = pos.float()[:, None] * inv_freq[None, :]
    ang = torch.cat((ang, ang), -1)
    cos, sin = ang.cos().half().float()[None, :, None], ang.sin().half().float()[None, :, None]
    q4, k4 = q.float().reshape(B, T, nh, hd), k.float().reshape(B, T, nkv, hd)
    q_ref = q4 * cos + _rot_half(q4) * sin
    k_ref = k4 * cos + _rot_half(k4) * sin
    glue.rope_append(q, k, v, kc, vc, pos, inv_freq, B)
    assert float((q.float().reshape(B, T, nh, hd) - q_ref).abs().max()) <= 4e-3
    assert float((kc[:, :, 40:40 + T].float() - k_ref.transpose(1, 2)).abs().max()) <= 4e-3
    assert torch.equal(vc[:, :, 40:40 + T], v.reshape(B, T, nkv, hd).transpose(1, 2))
    assert float(kc[:, :, :40].abs().max()) == 0 and float(kc[:, :, 40 + T:].abs().max()) == 0


@pytest.mark.parametrize("B,T,nh,nkv,hd,max_len,p0", [
    (1, 1, 32, 32, 128, 640, 512), (1, 1, 32, 32, 128, 640, 0), (2, 2, 8, 2, 64, 300, 100),
    (1, 1, 4, 4, 128, 5000, 4999), (1, 3, 64, 8, 128, 1100, 1024), (8, 1, 64, 8, 128, 1100, 1024)])
def test_decode_attention(B, T, nh, nkv, hd, max_len, p0):
    from eptq_b200.kernels import glue
    g = torch.Generator(device="cuda").manual_seed(p0 + nh)
    q = torch.randn(B * T, nh * hd, generator=g, device="cuda").half()
    kc = torch.randn(B, nkv, max_len, hd, generator=g, device="cuda").half()
    vc = torch.randn(B, nkv, max_len, hd, generator=g, device="cuda").half()
    pos = torch.arange(p0, p0 + T, device="cuda")
    for _ in range(2):                                            # second call: counters were left at zero
        out = glue.decode_attention(q, kc, vc, pos, B)
    qh = q.float().reshape(B, T, nh, hd).transpose(1, 2)
    kf = kc.float().repeat_interleave(nh // nkv, dim=1)
    vf = vc.float().repeat_interleave(nh // nkv, dim=1)
    mask = (torch.arange(max_len, device="cuda")[None, :] <= pos[:, None])[None, None]
    ref = F.scaled_dot_product_attention(qh, kf, vf, attn_mask=mask).transpose(1, 2).reshape(B * T, nh * hd)
    assert float((out.float() - ref).abs().max()) <= 3e-3 * max(1.0, float(ref.abs().max()))


@pytest.mark.parametrize("B,V,H,norm", [(1, 32000, 4096, True), (2, 1000, 512, False), (4, 517, 256, True)])
def test_lm_head_argmax_matches_torch(B, V, H, norm):
    """Fused final norm + fp16 projection + greedy pick against the same steps in PyTorch (fp32 matmul of the
    fp16 operands, logits rounded to fp16, first index of the maximum)."""
    from eptq_b200.kernels import glue
    g = torch.Generator(device="cuda").manual_seed(B * 1000 + V)
    W = (0.05 * torch.randn(V, H, generator=g, device="cuda")).half()
    x = torch.randn(B, H, generator=g, device="cuda").half()
    w = (1 + 0.1 * torch.randn(H, generator=g, device="cuda")).half() if norm else None
    eps = 1e-5
    hn = x
    if norm:
        xf = x.float()
        hn = w * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).half()
    want_logits = (hn.float() @ W.float().T)
    for _ in range(2):                                    # twice: the ticket in scratch must come back to zero
        tokens, logits = glue.lm_head_argmax(x, W, w, eps, want_logits=True)
        torch.cuda.synchronize()
        assert float((logits.float() - want_logits).abs().max()) <= 2e-3 * float(want_logits.abs().max())
        # the pick is the first maximum of the kernel's own fp16 logits, and a maximum of the reference within rounding
        assert torch.equal(tokens, logits.float().argmax(dim=-1))
        picked = want_logits.gather(1, tokens[:, None])[:, 0]
        assert bool((want_logits.max(dim=-1).values - picked <= 2e-3 * want_logits.abs().max()).all())
        t2, none = glue.lm_head_argmax(x, W, w, eps)
        assert none is None and torch.equal(t2, tokens)


def test_lm_head_argmax_always_names_a_vocabulary_row():
    """Non-finite activations (a model that overflowed) still give a token inside the vocabulary, picked like
    torch.argmax does: a NaN logit ranks above every number, ties go to the lower index."""
    from eptq_b200.kernels import glue
    g = torch.Generator(device="cuda").manual_seed(5)
    V, H = 3000, 512
    W = (0.05 * torch.randn(V, H, generator=g, device="cuda")).half()
    x = torch.randn(2, H, generator=g, device="cuda").half()
    x[0, 7] = float("nan")                                  # every logit of row 0 becomes NaN
    x[1, 3] = float("inf")                                  # +-inf logits in row 1 (NaN where the weight is 0)
    tokens, logits = glue.lm_head_argmax(x, W, None, 1e-5, want_logits=True)
    torch.cuda.synchronize()
    assert bool(((tokens >= 0) & (tokens < V)).all())
    assert torch.equal(tokens, logits.float().argmax(dim=-1))
    assert int(tokens[0]) == 0
