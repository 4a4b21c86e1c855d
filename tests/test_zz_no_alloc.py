"""The entry point with built-in scratch, for callers that cannot allocate device memory (a server
with fully pre-reserved memory, a plug-in inside another runtime's allocator): through the C ABI its
output must equal the regular entry point's, call after call, and oversized requests are refused.
Collected last on purpose, so that a failure here cannot hide results of the other tests."""
import ctypes as C

import pytest
import torch

import oracle
from eptq_b200 import _lib
from eptq_b200.kernels import _make_desc
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.synthetic import make_activations, make_layer
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


def _layer(out_f, in_f, seed, with_oracle=False):
    qd = make_layer(out_f, in_f, seed=seed, outlier_frac=0.004, bias=True)
    lin = EPTQLinear.from_quantized_data(qd, torch.from_numpy(oracle.d4_table(1.75)), "e8_d4").to(DEV)
    desc = _make_desc(lin.quantizer_type, lin.Q, lin._codebook32, lin._codebook, lin.g, lin.h, lin.O_vals,
                      lin.O_col, lin.O_row_ptr, lin.bias, lin.S_group, lin.qb_size)
    if with_oracle:
        W16 = oracle.dequantize_layer(util.qld_arrays(qd), oracle.d4_table(1.75))
        return lin, desc, (W16, qd.bias.numpy())
    return lin, desc


@pytest.mark.parametrize("out_f,in_f,batch", [(4096, 4096, 1), (1024, 2752, 3), (11008, 4096, 2)])
def test_static_scratch_matches_regular_entry_point(out_f, in_f, batch):
    lib = _lib.load()
    lin, desc, (W16, bias) = _layer(out_f, in_f, seed=out_f + batch, with_oracle=True)
    stream = torch.cuda.current_stream().cuda_stream
    ws = torch.zeros(lib.eptq_workspace_bytes(out_f // 8, in_f, batch), dtype=torch.uint8, device=DEV)
    for call in range(2):                                   # two calls in a row share the built-in scratch
        x = make_activations(batch, in_f, seed=100 + call).to(DEV)
        y_ref = torch.empty(batch, out_f, dtype=torch.float16, device=DEV)
        y_new = torch.full((batch, out_f), float("nan"), dtype=torch.float16, device=DEV)
        assert lib.eptq_linear_forward(C.byref(desc), x.data_ptr(), y_ref.data_ptr(), batch,
                                       ws.data_ptr(), ws.numel(), stream) == 0
        assert lib.eptq_linear_forward_static_scratch(C.byref(desc), x.data_ptr(), y_new.data_ptr(), batch,
                                                      stream) == 0
        torch.cuda.synchronize()
        # both are fp32 accumulations of the same products in different orders: compare with the
        # output tolerance of the suite, max|a-b| / max|b| <= 2e-3
        err = float((y_new.float() - y_ref.float()).abs().max() / y_ref.float().abs().max())
        assert err <= util.REL_TOL, err
        # and against the oracle: fp32 product with the reconstructed fp16 weight
        want = oracle.linear_reference(x.cpu().numpy(), W16, bias)
        assert util.max_rel_err(y_new.float().cpu().numpy(), want) <= util.REL_TOL


def test_static_scratch_limits():
    lib = _lib.load()
    assert lib.eptq_static_scratch_bytes() == 4 << 20
    stream = torch.cuda.current_stream().cuda_stream
    lin, desc = _layer(28672, 8192, seed=5)                 # Llama-2-70B gate shape
    x = make_activations(4, 8192, seed=1).to(DEV)
    y = torch.empty(4, 28672, dtype=torch.float16, device=DEV)
    assert lib.eptq_workspace_bytes(28672 // 8, 8192, 4) > lib.eptq_static_scratch_bytes()
    st = lib.eptq_linear_forward_static_scratch(C.byref(desc), x.data_ptr(), y.data_ptr(), 4, stream)
    assert st == 5 and b"workspace" in lib.eptq_strerror(st)          # too large for the fixed array
    assert lib.eptq_linear_forward_static_scratch(C.byref(desc), x.data_ptr(), y.data_ptr(), 5, stream) == 7
    assert lib.eptq_linear_forward_static_scratch(None, x.data_ptr(), y.data_ptr(), 1, stream) == 1
