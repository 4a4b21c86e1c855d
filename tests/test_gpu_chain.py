"""Chained launch (eptq_linear_forward_chain): o_proj -> gate/up -> down of a decoder layer in one launch,
checked against an fp32 PyTorch statement of the same arithmetic on oracle-reconstructed weights.

Three cases: a small layer (fewer units than blocks in a phase, so some blocks sit a phase out), a Llama-2-7B-sized
layer with the residual stream updated in place, and the same layer with the residual stream alternating between
two buffers."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import qld_arrays

pytestmark = pytest.mark.gpu

EPS = 1e-5


def _layer(out_f, in_f, seed, table):
    from eptq_b200.kernels.linear import EPTQLinear
    from eptq_b200.synthetic import make_layer
    qd = make_layer(out_f, in_f, seed=seed, device="cpu", scale_sigma=0.05)
    qd.g = (qd.g.float() * 0.03).half()                 # keep the stack's activations O(1)
    W = torch.from_numpy(oracle.dequantize_layer(qld_arrays(qd), oracle.d4_table(1.75)).astype(np.float32))
    return EPTQLinear.from_quantized_data(qd, table, "e8_d4").cuda(), W.cuda()


@pytest.fixture(scope="module")
def table():
    from eptq_b200.quantizers import E8D4Quantizer
    return E8D4Quantizer(radius=1.75).codes.cuda()


def _reference(att, x, w_norm, Wo, Wg, Wu, Wd):
    """fp32 matmuls on the reconstructed fp16 weights, fp16 roundings where separate fp16 ops would round."""
    f16 = lambda t: t.half().float()                                        # noqa: E731
    x1 = f16(x.float() + f16(att.float() @ Wo.T))
    n = f16(x1 * torch.rsqrt(x1.pow(2).mean(-1, keepdim=True) + EPS))       # LlamaRMSNorm: round, then weight
    hn = f16(w_norm.float() * n)
    gate, up = f16(hn @ Wg.T), f16(hn @ Wu.T)
    act = f16(f16(torch.nn.functional.silu(gate)) * up)
    return f16(x1 + f16(act @ Wd.T)), gate, up


@pytest.mark.parametrize("H,F_,two_buffers", [(1024, 2816, False), (4096, 11008, False), (4096, 11008, True)])
def test_chain_o_gateup_down(table, H, F_, two_buffers):
    from eptq_b200 import _lib
    from eptq_b200.kernels import linear_forward_chain, workspace_status
    (o, Wo), (gate, Wg), (up, Wu), (down, Wd) = (_layer(H, H, 1, table), _layer(F_, H, 2, table),
                                                 _layer(F_, H, 3, table), _layer(H, F_, 4, table))
    gen = torch.Generator(device="cuda").manual_seed(5)
    att = torch.randn(1, H, generator=gen, device="cuda").half()
    x0 = torch.randn(1, H, generator=gen, device="cuda").half()
    w_norm = (1 + 0.1 * torch.randn(H, generator=gen, device="cuda")).half()
    want, want_gate, want_up = _reference(att, x0, w_norm, Wo, Wg, Wu, Wd)

    keep, descs = [], []
    for m, fold in ((o, False), (gate, True), (up, True), (down, False)):
        d = m.descriptor()
        if fold:                                          # the norm's column weight rides on h
            h2 = (m.h.float() * w_norm.float()).half().contiguous()
            keep.append(h2)
            d.h = h2.data_ptr()
        descs.append(d)
    for _ in range(2):                                    # twice: the scratch must come back clean
        x = x0.clone()
        xm = torch.empty_like(x) if two_buffers else x         # residual stream after the attention block
        gbuf = torch.empty(1, F_, device="cuda", dtype=torch.float16)
        ubuf = torch.empty_like(gbuf)

        def fus(x_op=_lib.X_PLAIN, y_op=_lib.Y_STORE, residual=None, x_aux=None):
            f = _lib.EptqFusion()
            f.x_op, f.y_op, f.norm_eps = x_op, y_op, EPS
            f.residual = None if residual is None else residual.data_ptr()
            f.x_aux = None if x_aux is None else x_aux.data_ptr()
            return f
        fz = [fus(y_op=_lib.Y_ADD_RESIDUAL, residual=x), fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM),
              fus(_lib.X_SILU_MUL, _lib.Y_ADD_RESIDUAL, residual=xm, x_aux=ubuf)]
        linear_forward_chain(descs, [0, 1, 1, 2], [att, xm, xm, gbuf], [0, F_, F_, 0], fz, ys=[xm, gbuf, ubuf, x])
        assert workspace_status(device="cuda") == 0
        tol = 2e-3
        for got, ref in ((gbuf, want_gate), (ubuf, want_up), (x, want)):
            err = float((got.float() - ref).abs().max()) / float(ref.abs().max())
            assert err <= tol, err


def test_chain_rejects_bad_phases(table):
    from eptq_b200 import _lib
    from eptq_b200.kernels import linear_forward_chain
    a, _ = _layer(256, 256, 7, table)
    b, _ = _layer(256, 256, 8, table)
    x = torch.zeros(1, 256, device="cuda", dtype=torch.float16)
    f = _lib.EptqFusion()
    with pytest.raises(RuntimeError):
        linear_forward_chain([a.descriptor(), b.descriptor()], [0, 2], [x, x], [256, 256], [f, f])
    with pytest.raises(RuntimeError):
        linear_forward_chain([a.descriptor(), b.descriptor()], [1, 1], [x, x], [256, 256], [f, f])
