"""Prefill path (batch > 16): tcgen05 dequantise + GEMM (tile-by-tile reconstruction below 1024 tokens, one
reconstruction into scratch followed by the dense GEMM from 1024 tokens on) against the oracle and an fp32 matmul
of the bit-exact reconstructed weight."""
import numpy as np
import pytest
import torch

import oracle
from eptq_b200.kernels import workspace_for
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.synthetic import make_activations, make_layer
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build(qd, kind, radius):
    return EPTQLinear.from_quantized_data(qd, torch.from_numpy(util.oracle_table(kind, radius)), kind).to(DEV)


def timeout_flag():
    """Status word of the GEMM in the current stream's scratch (non-zero = a bounded wait ran out)."""
    ws = workspace_for(torch.device(DEV, torch.cuda.current_device()), 4096)
    torch.cuda.synchronize()
    return int(ws[:4096].view(torch.int32)[1023].item())


@pytest.mark.parametrize("kind,radius", [("e8_d4", 1.75), ("e8_lattice", 1.6)])
@pytest.mark.parametrize("out_f,in_f,tokens,bias,qb", [
    (128, 64, 128, False, None), (256, 256, 128, True, None), (136, 72, 130, False, None),
    (1024, 4096, 256, False, 128), (4096, 1024, 17, True, None), (264, 2752, 300, True, 8),
    (512, 512, 2048, False, None), (2048, 512, 300, True, None), (4104, 256, 1000, False, 8),
    (4096, 4096, 1024, True, None), (1000, 4096, 1536, False, 8),          # 1024 tokens and more: reconstruct once + dense GEMM
])
def test_gemm_vs_oracle(kind, radius, out_f, in_f, tokens, bias, qb):
    qd = make_layer(out_f, in_f, seed=out_f + in_f + tokens, outlier_frac=0.004, bias=bias, qb_size=qb)
    x = make_activations(tokens, in_f, seed=3)
    lin = build(qd, kind, radius)
    y = lin(x.to(DEV))
    assert timeout_flag() == 0
    W16 = lin.dequantize()
    assert torch.equal(W16.cpu(), torch.from_numpy(oracle.dequantize_layer(util.qld_arrays(qd), util.oracle_table(kind, radius))))
    y_ref = x.to(DEV).float() @ W16.float().T
    if bias:
        y_ref = y_ref + lin.bias.float()
    err = float((y.float() - y_ref).abs().max() / y_ref.abs().max())
    assert err <= util.REL_TOL, err
    # the tensor cores multiply exact fp16 tiles with fp32 accumulation: only the fp16 output rounding remains
    assert err <= 1.0e-3, err


def test_llama3_8b_prefill_shape():
    """Configuration 4: k/v projection 1024x4096, E8-D4 r=1.75 with group scales qb=128, 2048 tokens."""
    qd = make_layer(1024, 4096, seed=42, qb_size=128)
    x = make_activations(2048, 4096, seed=43)
    lin = build(qd, "e8_d4", 1.75)
    y = lin(x.to(DEV)).float()
    assert timeout_flag() == 0
    y_ref = x.to(DEV).float() @ lin.dequantize().float().T
    assert float((y - y_ref).abs().max() / y_ref.abs().max()) <= 1.0e-3
    # linearity at full size
    y2 = lin((2 * x).to(DEV)).float()
    assert float((y2 - 2 * y).abs().max() / y2.abs().max()) <= 2e-3


def test_dense_and_fused_paths_agree():
    """The same long prefill with a scratch buffer that holds the fp16 weight (dense path) and with the first MiB
    only (tile-by-tile reconstruction): same fp16 weight, same K order, so the outputs agree to fp32 rounding."""
    import ctypes as C
    from eptq_b200 import _lib
    lib = _lib.load()
    qd = make_layer(2048, 1024, seed=77, outlier_frac=0.004, bias=True)
    lin = build(qd, "e8_d4", 1.75)
    x = make_activations(1280, 1024, seed=5).to(DEV)
    d = lin.descriptor()
    need = lib.eptq_layer_workspace_bytes(C.byref(d), 1280)
    assert need >= (1 << 20) + 2048 * 1024 * 2
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for size in (need, 1 << 20):
        ws = torch.zeros(size, dtype=torch.uint8, device=DEV)
        y = torch.empty(1280, 2048, dtype=torch.float16, device=DEV)
        st = lib.eptq_linear_forward(C.byref(d), x.data_ptr(), y.data_ptr(), 1280, ws.data_ptr(), size, stream)
        assert st == 0
        torch.cuda.synchronize()
        assert int(ws[:4096].view(torch.int32)[1023].item()) == 0
        outs.append(y)
    ref = x.float() @ lin.dequantize().float().T + lin.bias.float()
    for y in outs:
        assert float((y.float() - ref).abs().max() / ref.abs().max()) <= 1.0e-3
    assert float((outs[0].float() - outs[1].float()).abs().max() / ref.abs().max()) <= 1.0e-3
