"""Fused prologue / epilogues of the group GEMV (eptq_linear_forward_group_fused) against the same
work done by separate calls, and against an fp32 PyTorch statement on oracle-reconstructed weights."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import qld_arrays

pytestmark = pytest.mark.gpu
_ORACLE_W = {}


def _layer(out_f, in_f, seed, table):
    from eptq_b200.kernels.linear import EPTQLinear
    from eptq_b200.synthetic import make_layer
    qd = make_layer(out_f, in_f, seed=seed, device="cpu")
    lin = EPTQLinear.from_quantized_data(qd, _cpu_table(table), "e8_d4").cuda()
    _ORACLE_W[id(lin)] = torch.from_numpy(oracle.dequantize_layer(qld_arrays(qd), oracle.d4_table(1.75)).astype(np.float32)).cuda()
    return lin


_CPU_TABLE = {}


def _cpu_table(table):
    """One CPU copy of the table for all layers of this module: layers of one launch must share a codebook."""
    if "t" not in _CPU_TABLE:
        _CPU_TABLE["t"] = table.cpu()
    return _CPU_TABLE["t"]


def _oracle_w(lin):
    """fp32 copy of the fp16 weight the reference's dequantize_layer gives for this layer."""
    return _ORACLE_W[id(lin)]


@pytest.fixture(scope="module")
def table():
    from eptq_b200.quantizers import E8D4Quantizer
    return E8D4Quantizer(radius=1.75).codes.cuda()


def _close(a, b, tol=2e-3):
    a, b = a.float(), b.float()
    return float((a - b).abs().max()) <= tol * max(float(b.abs().max()), 1e-6)


@pytest.mark.parametrize("B", [1, 2])
def test_fused_rmsnorm_and_residual(table, B):
    from eptq_b200 import _lib
    from eptq_b200.kernels import glue, h_absmax, linear_forward_group
    lins = [_layer(512, 1024, 1, table), _layer(256, 1024, 2, table)]
    g = torch.Generator(device="cuda").manual_seed(9)
    x = (3 * torch.randn(B, 1024, generator=g, device="cuda")).half()
    w = (1 + 0.2 * torch.randn(1024, generator=g, device="cuda")).half()
    res = torch.randn(B, 512, generator=g, device="cuda").half()
    hn = glue.add_rmsnorm(x.clone(), w, 1e-5)
    want0 = res + lins[0](hn)
    want1 = lins[1](hn)
    descs, keep, fz = [], [], []
    for i, m in enumerate(lins):
        h2 = (m.h.float() * w.float()).half().contiguous()
        d = m.descriptor()
        d.h, d.h_absmax = h2.data_ptr(), h_absmax(h2)
        keep.append(h2)
        descs.append(d)
        f = _lib.EptqFusion()
        f.x_op, f.norm_eps = _lib.X_RMSNORM, 1e-5
        f.y_op = _lib.Y_ADD_RESIDUAL if i == 0 else _lib.Y_STORE
        f.residual = res.data_ptr() if i == 0 else None
        fz.append(f)
    for _ in range(2):
        y0, y1 = linear_forward_group(descs, [x, x], [512, 256], fusions=fz)
    assert _close(y0, want0) and _close(y1, want1)
    # the same in fp32 PyTorch on the oracle's weights: LlamaRMSNorm (round, then weight), fp32 matmul
    xf = x.float()
    hn32 = (w.float() * (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-5)).half().float()).half().float()
    assert _close(y0, (res.float() + (hn32 @ _oracle_w(lins[0]).T).half().float()).half())
    assert _close(y1, (hn32 @ _oracle_w(lins[1]).T).half())
    # in place: the residual stream is the output
    stream = res.clone()
    f = _lib.EptqFusion()
    f.x_op, f.norm_eps, f.y_op, f.residual = _lib.X_RMSNORM, 1e-5, _lib.Y_ADD_RESIDUAL, stream.data_ptr()
    linear_forward_group(descs[:1], [x], [0], fusions=[f], ys=[stream])
    assert _close(stream, want0)


@pytest.mark.parametrize("B", [1, 2])
def test_fused_rope_and_cache(table, B):
    from eptq_b200 import _lib
    from eptq_b200.kernels import glue, linear_forward_group
    nh, nkv, hd, max_len, pos0 = 4, 2, 128, 40, 17
    q_l, k_l, v_l = _layer(nh * hd, 256, 3, table), _layer(nkv * hd, 256, 4, table), _layer(nkv * hd, 256, 5, table)
    g = torch.Generator(device="cuda").manual_seed(11)
    x = torch.randn(B, 256, generator=g, device="cuda").half()
    pos = torch.tensor([pos0], device="cuda")
    inv_freq = (1.0 / (10000.0 ** (torch.arange(0, hd, 2, device="cuda").float() / hd))).contiguous()
    # separate calls
    q, k, v = q_l(x), k_l(x), v_l(x)
    kc = torch.zeros(B, nkv, max_len, hd, device="cuda", dtype=torch.float16)
    vc = torch.zeros_like(kc)
    glue.rope_append(q, k, v, kc, vc, pos, inv_freq, B)
    # fused
    kc2, vc2 = torch.zeros_like(kc), torch.zeros_like(vc)
    fz = []
    for op in (_lib.Y_ROPE, _lib.Y_ROPE_TO_CACHE, _lib.Y_TO_CACHE):
        f = _lib.EptqFusion()
        f.x_op, f.y_op, f.rope_scaling, f.max_len = _lib.X_PLAIN, op, 1.0, max_len
        f.position, f.inv_freq = pos.data_ptr(), inv_freq.data_ptr()
        fz.append(f)
    q2 = linear_forward_group([q_l.descriptor(), k_l.descriptor(), v_l.descriptor()], [x, x, x],
                              [nh * hd, 0, 0], fusions=fz, ys=[None, kc2, vc2])[0]
    assert _close(q2, q, 3e-3)
    assert _close(kc2, kc, 3e-3) and _close(vc2, vc, 3e-3)
    # against fp32 PyTorch on the oracle's weights: rotary embedding with fp16 cos/sin, pairs (i, i + 64)
    ang = float(pos0) * inv_freq
    cos = torch.cat((ang.cos(), ang.cos())).half().float()
    sin = torch.cat((ang.sin(), ang.sin())).half().float()

    def rot(t, heads):
        t = t.float().reshape(B, heads, hd)
        half = torch.cat((-t[..., hd // 2:], t[..., :hd // 2]), dim=-1)
        return (t * cos + half * sin).reshape(B, heads * hd)
    xq = x.float()
    assert _close(q2, rot((xq @ _oracle_w(q_l).T).half(), nh), 3e-3)
    assert _close(kc2[:, :, pos0].reshape(B, -1), rot((xq @ _oracle_w(k_l).T).half(), nkv), 3e-3)
    assert _close(vc2[:, :, pos0].reshape(B, -1), (xq @ _oracle_w(v_l).T).half(), 3e-3)
    assert float(kc2[:, :, :pos0].abs().max()) == 0 and float(kc2[:, :, pos0 + 1:].abs().max()) == 0
