"""Several independent layers in one launch (eptq_linear_forward_group) against the oracle."""
import numpy as np
import pytest
import torch

import oracle
from eptq_b200.kernels.linear import EPTQLinear, forward_group
from eptq_b200.synthetic import make_activations, make_layer
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda"
TABLE = torch.from_numpy(oracle.d4_table(1.75))


def reference(qd, x):
    W16 = oracle.dequantize_layer(util.qld_arrays(qd), oracle.d4_table(1.75))
    return oracle.linear_reference(x.cpu().numpy(), W16, None if qd.bias is None else qd.bias.numpy())


@pytest.mark.parametrize("batch", [1, 2])
@pytest.mark.parametrize("shapes", [
    [(4096, 4096)] * 3,                                   # q, k, v
    [(11008, 4096), (11008, 4096)],                       # gate, up
    [(4096, 4096), (1024, 4096), (1024, 4096)],           # grouped-query attention
    [(40, 96), (8, 32), (264, 2752), (136, 160)],         # ragged row counts, tiny layers
    [(4096, 11008)],
    [(4096, 4096)] * 4 + [(11008, 4096)] * 2 + [(4096, 11008)],   # a whole decoder layer's linears
])
def test_group_matches_oracle(shapes, batch):
    qds = [make_layer(o, i, seed=11 * k + o + i, outlier_frac=0.004, bias=(k % 2 == 0)) for k, (o, i) in enumerate(shapes)]
    lins = [EPTQLinear.from_quantized_data(qd, TABLE, "e8_d4").to(DEV) for qd in qds]
    xs = [make_activations(batch, i, seed=31 + k) for k, (_, i) in enumerate(shapes)]
    ys = forward_group(lins, [x.to(DEV) for x in xs])
    for qd, x, y in zip(qds, xs, ys):
        assert util.max_rel_err(y.float().cpu().numpy(), reference(qd, x)) <= util.REL_TOL


def test_group_equals_single_calls_and_repeats():
    shapes = [(4096, 4096), (11008, 4096), (4096, 11008)]
    lins = [EPTQLinear.from_quantized_data(make_layer(o, i, seed=o + i), TABLE, "e8_d4").to(DEV) for o, i in shapes]
    xs = [make_activations(1, i, seed=i).to(DEV) for _, i in shapes]
    singles = [lin(x) for lin, x in zip(lins, xs)]
    first = forward_group(lins, xs)
    for a, b in zip(first, singles):
        assert float((a.float() - b.float()).abs().max() / b.float().abs().max()) <= util.REL_TOL
    # The partial sums of a row tile meet through fp32 atomic adds, whose order is not fixed: repeats agree
    # to fp32 rounding, i.e. at most an fp16 ulp apart, and the scratch is left clean every time.
    for _ in range(3):
        for a, b in zip(forward_group(lins, xs), first):
            assert float((a.float() - b.float()).abs().max() / b.float().abs().max()) <= 1e-3


def test_group_rejects_ineligible_sets():
    e8 = EPTQLinear.from_quantized_data(make_layer(64, 64, seed=1), torch.from_numpy(oracle.e8_table(1.6)), "e8_lattice").to(DEV)
    d4 = EPTQLinear.from_quantized_data(make_layer(64, 64, seed=1), TABLE, "e8_d4").to(DEV)
    with pytest.raises(RuntimeError):                                  # one codebook per launch
        forward_group([e8, d4], [make_activations(1, 64).to(DEV)] * 2)
    scaled = EPTQLinear.from_quantized_data(make_layer(256, 64, seed=2, qb_size=128), TABLE, "e8_d4").to(DEV)
    with pytest.raises(RuntimeError):                                  # group scales run on the general kernel
        forward_group([scaled], [make_activations(1, 64).to(DEV)])
    with pytest.raises(RuntimeError):
        forward_group([d4], [make_activations(17, 64).to(DEV)])       # above 16 rows the layers are GEMMs


@pytest.mark.parametrize("batch", [3, 4, 7, 16])
def test_group_batches_above_two(batch):
    """Batches 3..16 run as passes of two rows over the same weights."""
    shapes = [(4096, 4096), (264, 2752), (1024, 4096)]
    qds = [make_layer(o, i, seed=5 * k + o, outlier_frac=0.004, bias=(k == 0)) for k, (o, i) in enumerate(shapes)]
    lins = [EPTQLinear.from_quantized_data(qd, TABLE, "e8_d4").to(DEV) for qd in qds]
    xs = [make_activations(batch, i, seed=51 + k) for k, (_, i) in enumerate(shapes)]
    ys = forward_group(lins, [x.to(DEV) for x in xs])
    for qd, x, y in zip(qds, xs, ys):
        ref = reference(qd, x)
        for b in range(batch):
            assert util.max_rel_err(y[b].float().cpu().numpy(), ref[b]) <= util.REL_TOL
    y1 = lins[0](xs[0].to(DEV))                       # the single-layer entry takes the same route
    assert util.max_rel_err(y1.float().cpu().numpy(), reference(qds[0], xs[0])) <= util.REL_TOL


@pytest.mark.parametrize("B", [1, 2])
def test_e8_group_matches_oracle(B):
    """E8 layers: packed table partly in shared memory, partly read through L2."""
    e8 = oracle.e8_table(1.6)
    table = torch.from_numpy(e8)
    shapes = [(4096, 4096), (1024, 2048), (2048, 11008), (64, 64)]
    qds = [make_layer(o, i, seed=3 * o + i, bias=(k == 1)) for k, (o, i) in enumerate(shapes)]
    lins = [EPTQLinear.from_quantized_data(qd, table, "e8_lattice").to(DEV) for qd in qds]
    xs = [make_activations(B, i, seed=i + 7) for _, i in shapes]

    def ref(qd, x):
        W16 = oracle.dequantize_layer(util.qld_arrays(qd), e8)
        return oracle.linear_reference(x.numpy(), W16, None if qd.bias is None else qd.bias.numpy())
    for _ in range(2):
        ys = forward_group(lins, [x.to(DEV) for x in xs])
    for qd, x, y in zip(qds, xs, ys):
        assert util.max_rel_err(y.float().cpu().numpy(), ref(qd, x)) <= util.REL_TOL
    # the single-layer entry point takes the same kernel for a layer this large
    y0 = lins[0](xs[0].to(DEV))
    assert util.max_rel_err(y0.float().cpu().numpy(), ref(qds[0], xs[0])) <= util.REL_TOL
