"""E8-D4 at batch 1 through EPTQLinear against the oracle, over shapes that land in each kernel behind it:
the streaming kernel (N a multiple of 64), the group kernel (N a multiple of 32 only) and the general SIMT
kernel (ragged N, tiny layers).  The per-layer tensor-core kernel of the static-scratch entry point has its
own oracle comparison in test_zz_no_alloc.py."""
import numpy as np
import pytest
import torch

import oracle
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.synthetic import make_activations, make_layer
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build(qd):
    return EPTQLinear.from_quantized_data(qd, torch.from_numpy(oracle.d4_table(1.75)), "e8_d4").to(DEV)


def reference(qd, x):
    W16 = oracle.dequantize_layer(util.qld_arrays(qd), oracle.d4_table(1.75))
    return oracle.linear_reference(x.cpu().numpy(), W16, None if qd.bias is None else qd.bias.numpy())


@pytest.mark.parametrize("out_f,in_f", [
    (8, 32), (16, 32), (40, 96), (128, 128), (136, 160), (264, 2752), (2048, 1024), (1024, 8192),
    (11008, 4096), (4096, 11008), (4096, 4096), (14336, 4096), (1024, 4096), (768, 3072), (50 * 8, 64),
])
@pytest.mark.parametrize("bias", [False, True])
def test_shapes(out_f, in_f, bias):
    qd = make_layer(out_f, in_f, seed=out_f * 7 + in_f, outlier_frac=0.004, bias=bias)
    x = make_activations(1, in_f, seed=11)
    y = build(qd)(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, reference(qd, x)) <= util.REL_TOL


@pytest.mark.parametrize("scale", [1e-4, 1e-2, 30.0, 200.0])
def test_activation_magnitudes(scale):
    """The scaling of the activations (two int8 digits of x*h / max|x*h|) keeps precision whatever the magnitude of x."""
    qd = make_layer(1024, 2048, seed=3)
    x = (make_activations(1, 2048, seed=12).float() * scale).half()
    y = build(qd)(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, reference(qd, x)) <= util.REL_TOL


def test_sparse_and_spiky_activations():
    qd = make_layer(512, 4096, seed=4)
    x = make_activations(1, 4096, seed=13)
    x[0, ::3] = 0
    x[0, 100] = 300.0            # one dominant channel inside a block of ordinary values
    x[0, 3000:3200] = 0          # a column block that is entirely zero
    y = build(qd)(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, reference(qd, x)) <= util.REL_TOL
    z = build(qd)(torch.zeros(1, 4096, dtype=torch.float16, device=DEV))
    assert float(z.abs().max()) == 0.0


@pytest.mark.parametrize("frac", [0.0, 0.1, 1.0])
def test_marker_density(frac):
    qd = make_layer(256, 512, seed=5, outlier_frac=frac, bias=True)
    x = make_activations(1, 512, seed=14)
    y = build(qd)(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, reference(qd, x)) <= util.REL_TOL


@pytest.mark.parametrize("batch", [2, 3, 4])
@pytest.mark.parametrize("out_f,in_f", [(4096, 4096), (264, 2752), (11008, 4096), (4096, 11008), (40, 96)])
def test_small_batches(batch, out_f, in_f):
    """Batches 2..4 run in the group kernel (two batch rows per pass)."""
    qd = make_layer(out_f, in_f, seed=out_f + in_f + batch, outlier_frac=0.004, bias=True)
    x = make_activations(batch, in_f, seed=21)
    x[batch - 1] *= 37.0                      # rows with very different magnitudes get their own scale
    y = build(qd)(x.to(DEV)).float().cpu().numpy()
    ref = reference(qd, x)
    for b in range(batch):
        assert util.max_rel_err(y[b], ref[b]) <= util.REL_TOL


def test_agrees_with_general_kernel_and_is_repeatable():
    """Five identical rows (three passes of two rows) agree with the single row."""
    qd = make_layer(4096, 4096, seed=6)
    lin = build(qd)
    x = make_activations(1, 4096, seed=15).to(DEV)
    y1 = lin(x)
    y2 = lin(torch.cat([x, x, x, x, x]))
    ref = y2[0].float()
    assert float((y1[0].float() - ref).abs().max() / ref.abs().max()) <= util.REL_TOL
    for _ in range(3):                               # batch 1: fp32 atomic adds, repeats agree to an fp16 ulp
        assert util.max_rel_err(lin(x).float().cpu().numpy(), y1.float().cpu().numpy()) <= 1e-3
    x4 = torch.cat([x, x, x, x])                     # batch 4: two passes of the same kernel
    y4 = lin(x4)
    for _ in range(3):
        assert util.max_rel_err(lin(x4).float().cpu().numpy(), y4.float().cpu().numpy()) <= 1e-3


def test_interleaved_shapes_share_scratch():
    """Layers of different shapes called back to back on one stream reuse one scratch buffer."""
    shapes = [(4096, 4096), (11008, 4096), (4096, 11008), (264, 2752)]
    lins = [build(make_layer(o, i, seed=o + i)) for o, i in shapes]
    xs = [make_activations(1, i, seed=i).to(DEV) for _, i in shapes]
    first = [lin(x) for lin, x in zip(lins, xs)]
    for _ in range(3):
        for lin, x, y0 in zip(lins, xs, first):
            assert util.max_rel_err(lin(x).float().cpu().numpy(), y0.float().cpu().numpy()) <= 1e-3
    g = torch.cuda.CUDAGraph()
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        outs = [lin(x) for lin, x in zip(lins, xs)]
        torch.cuda.synchronize()
        with torch.cuda.graph(g, stream=side):
            outs = [lin(x) for lin, x in zip(lins, xs)]
    g.replay()
    torch.cuda.synchronize()
    for y, y0 in zip(outs, first):
        assert util.max_rel_err(y.float().cpu().numpy(), y0.float().cpu().numpy()) <= 1e-3
