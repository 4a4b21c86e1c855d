"""torch.compile(fullgraph=True) over the custom ops and over EPTQLinear modules: the ops are registered with
fake implementations so that the compiler treats each as one opaque op, as the reference's are
(kernels/__init__.py:46-91, bench_decode.py:146-157)."""
import numpy as np
import pytest
import torch

import oracle
from tests.util import REL_TOL, max_rel_err, qld_arrays

pytestmark = pytest.mark.gpu


def _layer(out_f, in_f, seed):
    from eptq_b200.kernels.linear import EPTQLinear
    from eptq_b200.quantizers import E8D4Quantizer
    from eptq_b200.synthetic import make_layer
    qd = make_layer(out_f, in_f, seed=seed)
    W16 = oracle.dequantize_layer(qld_arrays(qd), oracle.d4_table(1.75)).astype(np.float32)
    lin = EPTQLinear.from_quantized_data(qd, E8D4Quantizer(radius=1.75).codes, "e8_d4").cuda()
    return lin, W16


def test_compiled_two_layer_module_matches_oracle():
    a, Wa = _layer(512, 256, 21)
    b, Wb = _layer(256, 512, 22)

    class Two(torch.nn.Module):
        def __init__(self):
            super().__init__()
            self.a, self.b = a, b

        def forward(self, x):
            return self.b(torch.nn.functional.silu(self.a(x)))

    mod = Two()
    x = torch.randn(1, 256, generator=torch.Generator().manual_seed(1)).half().cuda()
    eager = mod(x)
    compiled = torch.compile(mod, fullgraph=True)
    got = compiled(x)
    # the accumulation order of the GEMV's partial sums is not fixed and the compiler fuses silu: not bit-equal
    assert max_rel_err(got.float().cpu().numpy(), eager.float().cpu().numpy()) <= REL_TOL
    h = torch.nn.functional.silu(torch.from_numpy(x.float().cpu().numpy() @ Wa.T).half().float())
    want = h.numpy() @ Wb.T
    assert max_rel_err(got.float().cpu().numpy(), want) <= 2 * REL_TOL       # two layers, two roundings


def test_compiled_e8d4_forward_op():
    from eptq_b200.kernels import e8d4_forward
    lin, W = _layer(384, 256, 23)
    x = torch.randn(2, 256, generator=torch.Generator().manual_seed(2)).half().cuda()
    empty = torch.empty(0, dtype=torch.float16, device="cuda")

    def f(x):
        return e8d4_forward(lin.Q, lin._codebook, lin.g, lin.h, x, lin.O_vals, lin.O_col, lin.O_row_ptr, empty) * 2

    got = torch.compile(f, fullgraph=True)(x)
    want = 2 * (x.float().cpu().numpy() @ W.T)
    assert max_rel_err(got.float().cpu().numpy(), want) <= REL_TOL
