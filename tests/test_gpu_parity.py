"""Parity of the CUDA path with the oracle, through the C ABI (needs a B200)."""
import numpy as np
import pytest
import torch

import oracle
from eptq_b200 import _lib
from eptq_b200.kernels import e8_forward, e8d4_forward
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.synthetic import LLAMA2_7B_LINEARS, make_activations, make_layer
from tests import util

pytestmark = pytest.mark.gpu
DEV = "cuda"


def build_linear(qd, kind, radius):
    tab = torch.from_numpy(util.oracle_table(kind, radius))
    return EPTQLinear.from_quantized_data(qd, tab, kind).to(DEV)


def oracle_outputs(qd, kind, radius, x):
    W16 = oracle.dequantize_layer(util.qld_arrays(qd), util.oracle_table(kind, radius))
    bias = None if qd.bias is None else qd.bias.numpy()
    return W16, oracle.linear_reference(x.cpu().numpy(), W16, bias)


@pytest.mark.parametrize("name", util.CASES)
def test_golden_dequantize_bit_exact(name):
    d = util.load_case(name)
    lin = build_linear(util.case_qld(d), d["kind"], d["radius"])
    W = lin.dequantize().cpu().numpy()
    assert np.array_equal(W.view(np.uint16), d["W16"].view(np.uint16))


@pytest.mark.parametrize("name", util.CASES)
def test_golden_layer_outputs(name):
    d = util.load_case(name)
    lin = build_linear(util.case_qld(d), d["kind"], d["radius"])
    y = lin(torch.from_numpy(d["x"]).to(DEV)).float().cpu().numpy()
    assert y.shape == d["y"].shape
    assert util.max_rel_err(y, d["y"]) <= util.REL_TOL


def test_config1_full_size():
    """OPT-125m fc1, E8 r=1.6, seed 42: weight digest from the reference, output vs oracle."""
    ref = util.load_json("config1.json")
    qd = make_layer(ref["out"], ref["in"], seed=ref["seed"])
    lin = build_linear(qd, "e8_lattice", ref["radius"])
    assert util.sha(lin.dequantize()) == ref["W16_sha256"]
    x = make_activations(1, ref["in"], seed=42)
    _, y_ref = oracle_outputs(qd, "e8_lattice", ref["radius"], x)
    assert abs(float(np.abs(y_ref).max()) - ref["y_abs_max"]) < 1e-2
    y = lin(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, y_ref) <= util.REL_TOL


def test_config2_qproj_weight_digest():
    ref = util.load_json("config2_qproj.json")
    qd = make_layer(ref["out"], ref["in"], seed=ref["seed"])
    assert util.sha(qd.Q) == ref["Q_sha256"]
    lin = build_linear(qd, "e8_d4", ref["radius"])
    assert util.sha(lin.dequantize()) == ref["W16_sha256"]


@pytest.mark.parametrize("kind,radius", [("e8_d4", 1.75), ("e8_lattice", 1.6)])
@pytest.mark.parametrize("out_f,in_f", [(4096, 4096), (11008, 4096), (4096, 11008)])
@pytest.mark.parametrize("batch", [1, 4, 16])
def test_llama7b_shapes_vs_oracle(kind, radius, out_f, in_f, batch):
    qd = make_layer(out_f, in_f, seed=42)
    x = make_activations(batch, in_f, seed=43)
    W16, y_ref = oracle_outputs(qd, kind, radius, x)
    lin = build_linear(qd, kind, radius)
    assert torch.equal(lin.dequantize().cpu(), torch.from_numpy(W16))
    y = lin(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, y_ref) <= util.REL_TOL


@pytest.mark.parametrize("kind,radius", [("e8_d4", 1.75), ("e8_lattice", 1.6)])
@pytest.mark.parametrize("out_f,in_f,batch,bias,qb", [
    (8, 8, 1, False, None), (8, 7, 2, True, None), (40, 33, 3, False, None), (24, 264, 5, True, None),
    (64, 1000, 7, False, 32), (136, 520, 16, True, 8), (1032, 2056, 2, False, None), (16, 8192, 1, True, 16),
    (256, 96, 33, False, 128), (4096, 64, 1, False, None),
])
def test_ragged_and_edge_shapes(kind, radius, out_f, in_f, batch, bias, qb):
    qd = make_layer(out_f, in_f, seed=out_f + in_f, outlier_frac=0.01, bias=bias, qb_size=qb)
    x = make_activations(batch, in_f, seed=5)
    W16, y_ref = oracle_outputs(qd, kind, radius, x)
    lin = build_linear(qd, kind, radius)
    assert torch.equal(lin.dequantize().cpu(), torch.from_numpy(W16))
    y = lin(x.to(DEV)).float().cpu().numpy()
    assert util.max_rel_err(y, y_ref) <= util.REL_TOL


@pytest.mark.parametrize("frac", [0.0, 0.05, 0.5, 1.0])
def test_marker_density(frac):
    qd = make_layer(64, 512, seed=17, outlier_frac=frac)
    x = make_activations(2, 512, seed=6)
    W16, y_ref = oracle_outputs(qd, "e8_d4", 1.75, x)
    lin = build_linear(qd, "e8_d4", 1.75)
    assert torch.equal(lin.dequantize().cpu(), torch.from_numpy(W16))
    assert util.max_rel_err(lin(x.to(DEV)).float().cpu().numpy(), y_ref) <= util.REL_TOL


def test_reference_op_signatures():
    """e8_forward / e8d4_forward with the reference's nine positional tensors."""
    for kind, radius, op in (("e8_lattice", 1.6, e8_forward), ("e8_d4", 1.75, e8d4_forward)):
        qd = make_layer(128, 512, seed=3, outlier_frac=0.01)
        lin = build_linear(qd, kind, radius)
        x = make_activations(3, 512, seed=4).to(DEV)
        empty = torch.empty(0, dtype=torch.float16, device=DEV)
        y = op(lin.Q, lin._codebook, lin.g, lin.h, x, lin.O_vals, lin.O_col, lin.O_row_ptr, empty)
        assert y.shape == (3, 128) and y.dtype == torch.float16 and y.device == x.device
        tab16 = util.oracle_table(kind, radius).astype(np.float16)
        y_formula = oracle.gemv_formula_reference(util.qld_arrays(qd), tab16, x.cpu().numpy())
        # The reference's own tests accept 0.05 absolute on unit-scale data (test_e8_cuda.py:106-110).
        assert np.abs(y.float().cpu().numpy() - y_formula).max() < 0.05
        assert util.max_rel_err(y.float().cpu().numpy(), y_formula) <= util.REL_TOL


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16])
def test_activation_dtypes_and_leading_shape(dtype):
    qd = make_layer(64, 256, seed=8, bias=True)
    lin = build_linear(qd, "e8_d4", 1.75)
    x = make_activations(6, 256, seed=9).to(DEV).to(dtype).reshape(2, 3, 256)
    y = lin(x)
    assert y.shape == (2, 3, 64) and y.dtype == dtype
    _, y_ref = oracle_outputs(qd, "e8_d4", 1.75, x.reshape(6, 256).half().cpu())
    assert util.max_rel_err(y.float().reshape(6, 64).cpu().numpy(), y_ref) <= 2 * util.REL_TOL


def test_non_contiguous_input_and_empty_batch():
    qd = make_layer(64, 256, seed=8)
    lin = build_linear(qd, "e8_d4", 1.75)
    xt = make_activations(256, 4, seed=9).to(DEV).t()            # (4, 256) non-contiguous view
    _, y_ref = oracle_outputs(qd, "e8_d4", 1.75, xt.contiguous().cpu())
    assert util.max_rel_err(lin(xt).float().cpu().numpy(), y_ref) <= util.REL_TOL
    assert lin(torch.empty(0, 256, dtype=torch.float16, device=DEV)).shape == (0, 64)


def test_linearity_at_full_size():
    """Size-independent property at a configuration-2 shape: f(a*x1 + x2) = a*f(x1) + f(x2)."""
    out_f, in_f = LLAMA2_7B_LINEARS["mlp.down_proj"]
    lin = build_linear(make_layer(out_f, in_f, seed=42, device="cpu"), "e8_d4", 1.75)
    x1 = make_activations(1, in_f, seed=1).to(DEV)
    x2 = make_activations(1, in_f, seed=2).to(DEV)
    y12 = lin((2 * x1 + x2)).float()
    ysum = 2 * lin(x1).float() + lin(x2).float()
    assert float((y12 - ysum).abs().max() / ysum.abs().max()) <= 2 * util.REL_TOL


def test_repeatable_and_workspace_left_clean():
    qd = make_layer(4096, 4096, seed=42)
    lin = build_linear(qd, "e8_d4", 1.75)
    x = make_activations(1, 4096, seed=1).to(DEV)
    ys = [lin(x) for _ in range(4)]
    for y in ys[1:]:             # fp32 atomic adds: the order varies, the result to an fp16 ulp does not
        assert float((y.float() - ys[0].float()).abs().max() / ys[0].float().abs().max()) <= 1e-3


def test_bad_arguments_raise():
    qd = make_layer(64, 256, seed=8)
    lin = build_linear(qd, "e8_d4", 1.75)
    with pytest.raises(RuntimeError):
        e8d4_forward(lin.Q, lin._codebook, lin.g, lin.h, torch.zeros(1, 255, dtype=torch.float16, device=DEV),
                     lin.O_vals, lin.O_col, lin.O_row_ptr, torch.empty(0, dtype=torch.float16, device=DEV))
    with pytest.raises(RuntimeError):
        e8d4_forward(lin.Q, lin._codebook, lin.g, lin.h, torch.zeros(1, 256, dtype=torch.float32, device=DEV),
                     lin.O_vals, lin.O_col, lin.O_row_ptr, torch.empty(0, dtype=torch.float16, device=DEV))
    lib = _lib.load()
    misaligned = lin.Q.data_ptr() + 2
    st = lib.eptq_e8d4_forward(misaligned, lin._codebook.data_ptr(), lin.g.data_ptr(), lin.h.data_ptr(),
                               lin.h.data_ptr(), None, None, lin.O_row_ptr.data_ptr(), None,
                               lin.g.data_ptr(), 8, 256, 1, None, 0, None)
    assert st == 3     # EPTQ_ERR_ALIGN, reported before any launch


def test_launch_counter_moves():
    qd = make_layer(64, 256, seed=8)
    lin = build_linear(qd, "e8_d4", 1.75)
    before = _lib.launch_count()
    lin(make_activations(1, 256).to(DEV))
    torch.cuda.synchronize()
    assert _lib.launch_count() == before + 1


def test_reference_signature_entry_reaches_streaming_kernel():
    """eptq_e8d4_forward takes exactly the reference's arguments (csrc/eptq_kernels.h:31-41); at batch 1 on a
    lattice table it must run the streaming kernel, not a side path, and match the oracle.  The Python
    e8_forward op must reach the persistent E8 kernel likewise."""
    import ctypes as C
    import oracle
    from eptq_b200 import _lib
    from eptq_b200.kernels import e8_forward, workspace_for
    from eptq_b200.kernels.linear import EPTQLinear
    from eptq_b200.synthetic import make_activations, make_layer
    lib = _lib.load()
    qd = make_layer(4096, 4096, seed=77)
    lin = EPTQLinear.from_quantized_data(qd, torch.from_numpy(oracle.d4_table(1.75)), "e8_d4").cuda()
    x = make_activations(1, 4096, seed=3).cuda()
    y = torch.empty(1, 4096, dtype=torch.float16, device="cuda")
    ws = workspace_for(x.device, lib.eptq_workspace_bytes(512, 4096, 1))
    lib.eptq_forget_codebook(None)
    before = _lib.kernel_launch_count(_lib.KERNEL_GEMV_STREAM)
    st = lib.eptq_e8d4_forward(lin.Q.data_ptr(), lin._codebook.data_ptr(), lin.g.data_ptr(), lin.h.data_ptr(),
                               x.data_ptr(), lin.O_vals.data_ptr(), lin.O_col.data_ptr(), lin.O_row_ptr.data_ptr(),
                               None, y.data_ptr(), 512, 4096, 1, ws.data_ptr(), ws.numel(),
                               torch.cuda.current_stream().cuda_stream)
    assert st == 0
    torch.cuda.synchronize()
    assert _lib.kernel_launch_count(_lib.KERNEL_GEMV_STREAM) == before + 1
    W16 = oracle.dequantize_layer(util.qld_arrays(qd), oracle.d4_table(1.75))
    assert util.max_rel_err(y.float().cpu().numpy(), oracle.linear_reference(x.cpu().numpy(), W16, None)) <= util.REL_TOL
    # E8 through the Python op of the reference's signature
    qd8 = make_layer(4096, 4096, seed=78)
    tab8 = torch.from_numpy(oracle.e8_table(1.6))
    lin8 = EPTQLinear.from_quantized_data(qd8, tab8, "e8_lattice").cuda()
    before = _lib.kernel_launch_count(_lib.KERNEL_GEMV_GROUP)
    y8 = e8_forward(lin8.Q, lin8._codebook, lin8.g, lin8.h, x, lin8.O_vals, lin8.O_col, lin8.O_row_ptr,
                    torch.empty(0, dtype=torch.float16, device="cuda"))
    torch.cuda.synchronize()
    assert _lib.kernel_launch_count(_lib.KERNEL_GEMV_GROUP) == before + 1
    W8 = oracle.dequantize_layer(util.qld_arrays(qd8), oracle.e8_table(1.6))
    assert util.max_rel_err(y8.float().cpu().numpy(), oracle.linear_reference(x.cpu().numpy(), W8, None)) <= util.REL_TOL
