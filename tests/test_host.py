"""Host-side logic that needs no GPU: format round trip, codebooks, CSR build, error behaviour."""
import numpy as np
import pytest
import torch

import oracle
from eptq_b200 import QuantizedLayerData
from eptq_b200.kernels.linear import EPTQLinear
from eptq_b200.quantizers import E8D4Quantizer, E8LatticeQuantizer
from eptq_b200.synthetic import make_layer
from tests import util


def test_layer_data_round_trip(tmp_path):
    qd = make_layer(64, 48, seed=3, bias=True, qb_size=32)
    qd.chosen_r = 1.7
    qd.save(tmp_path / "l.pt")
    back = QuantizedLayerData.load(tmp_path / "l.pt")
    for k in ("Q", "g", "h", "O", "bias", "S_group"):
        assert torch.equal(getattr(qd, k), getattr(back, k))
    assert back.chosen_r == 1.7 and back.Q.device.type == "cpu"
    assert set(qd.to_dict()) == {"Q", "g", "h", "O", "bias", "chosen_r", "S_group"}
    assert set(make_layer(16, 8).to_dict()) == {"Q", "g", "h", "O"}


def test_product_tables_equal_oracle_tables():
    e8 = E8LatticeQuantizer(radius=1.6)
    e8.remove_last()
    assert np.array_equal(e8.points.numpy(), oracle.e8_table(1.6))
    d4 = E8D4Quantizer(radius=1.75)
    assert np.array_equal(d4.codes.numpy(), oracle.d4_table(1.75))
    d4.set_radius(1.9)
    assert np.array_equal(d4.codes.numpy(), oracle.d4_table(1.9))


@pytest.mark.parametrize("kind", ["e8_lattice", "e8_d4"])
def test_quantizer_dequant_matches_oracle_lookup(kind):
    qd = make_layer(32, 24, seed=5, outlier_frac=0.0)
    idx = qd.Q.int() + 32768
    if kind == "e8_lattice":
        q = E8LatticeQuantizer(radius=1.6)
        q.remove_last()
        tab = oracle.e8_table(1.6)
    else:
        q = E8D4Quantizer(radius=1.75)
        tab = oracle.d4_table(1.75)
    W = q.dequant(idx, 1.0).numpy()
    one = np.ones(32, np.float16)
    Wo = oracle.dequantize_layer(
        oracle.LayerArrays(Q=qd.Q.numpy(), g=one, h=np.ones(24, np.float16), O=qd.O.numpy()), tab)
    assert np.array_equal(W.astype(np.float16), Wo)


def test_linear_builds_csr_like_oracle():
    d = util.load_case("d4_marker_rows")
    lin = EPTQLinear.from_quantized_data(util.case_qld(d), torch.from_numpy(oracle.d4_table(1.75)), "e8_d4")
    col, ptr = oracle.csr_from_q(d["Q"])
    assert np.array_equal(lin.O_col.numpy(), col) and np.array_equal(lin.O_row_ptr.numpy(), ptr)
    assert lin.O_col.dtype == torch.int32 and lin.O_row_ptr.dtype == torch.int32
    assert lin.in_features == 19 and lin.out_features == 24
    assert lin._codebook.shape == (512, 4) and lin._codebook.dtype == torch.float16
    assert "n_masked=21" in lin.extra_repr()


def test_linear_rejects_inconsistent_O():
    qd = make_layer(32, 16, seed=1, outlier_frac=0.1)
    qd.O = qd.O[:-1]
    with pytest.raises(AssertionError):
        EPTQLinear.from_quantized_data(qd, torch.from_numpy(oracle.d4_table(1.75)), "e8_d4")


def test_codebook_is_shared_between_layers():
    tab = torch.from_numpy(oracle.d4_table(1.75))
    a = EPTQLinear.from_quantized_data(make_layer(16, 8, seed=1), tab, "e8_d4")
    b = EPTQLinear.from_quantized_data(make_layer(24, 8, seed=2), tab, "e8_d4")
    assert a._codebook is b._codebook and a._codebook32 is b._codebook32


def test_cpu_tensor_raises_instead_of_falling_back(built_library):
    lin = EPTQLinear.from_quantized_data(make_layer(16, 8, seed=1), torch.from_numpy(oracle.d4_table(1.75)), "e8_d4")
    with pytest.raises(RuntimeError, match="CUDA"):
        lin(torch.zeros(1, 8, dtype=torch.float16))
    from eptq_b200.kernels import e8d4_forward
    with pytest.raises(RuntimeError, match="CUDA"):
        e8d4_forward(lin.Q, lin._codebook, lin.g, lin.h, torch.zeros(1, 8, dtype=torch.float16),
                     lin.O_vals, lin.O_col, lin.O_row_ptr, torch.empty(0, dtype=torch.float16))


def test_e8_table_packs_and_unpacks():
    """The packed E8 table (4 bits per coordinate) reproduces the fp32 table; odd tables are refused."""
    import oracle
    from eptq_b200.kernels import pack_e8_table, unpack_e8_table
    t = torch.from_numpy(oracle.e8_table(1.6))
    word, scale = pack_e8_table(t)
    assert word.shape == (65536,) and word.dtype == torch.int32 and abs(scale - 1 / 1.6) < 1e-6
    back = unpack_e8_table(word, scale)
    assert float((back[:65535] - t).abs().max()) < 1e-6
    assert float(back[65535].abs().max()) == 0.0                 # marker slot decodes to zero
    assert pack_e8_table(t * (1 + 0.05 * t.abs())) is None       # radially warped: not a lattice multiple
    assert pack_e8_table(t[:, :4]) is None


def test_critical_lists_group_blocks_by_unit_and_check_their_range(built_library):
    """The per-unit lists of critical blocks are a permutation of the CSR side tables grouped by 64 x 128 unit,
    and a layer whose corrections could overflow the kernel's 32-bit fixed-point sums gets no lists."""
    from eptq_b200.kernels import CRIT_ROW_LIMIT, critical_lists
    qd = make_layer(1024, 512, seed=5, outlier_frac=0.01)
    lin = EPTQLinear.from_quantized_data(qd, torch.from_numpy(oracle.d4_table(1.75)), "e8_d4")
    M, N = lin.Q.shape
    ptr, pos, O = lin.crit_ptr, lin.crit_pos, lin.crit_O
    assert ptr is not None and int(ptr[-1]) == lin.O_col.shape[0] == pos.shape[0] == O.shape[0]
    cc = (N + 127) // 128
    assert ptr.shape[0] == ((M + 63) // 64) * cc + 1
    rows = torch.repeat_interleave(torch.arange(M), (lin.O_row_ptr[1:] - lin.O_row_ptr[:-1]).long())
    want = sorted(zip(((rows // 64) * cc + lin.O_col.long() // 128).tolist(), (rows % 64).tolist(), lin.O_col.tolist()))
    unit_of_entry = torch.repeat_interleave(torch.arange(ptr.shape[0] - 1), (ptr[1:] - ptr[:-1]).long())
    p = pos.long() & 0xFFFFFFFF
    got = sorted(zip(unit_of_entry.tolist(), (p >> 16).tolist(), (p & 0xFFFF).tolist()))
    assert got == want
    # the same O values, regrouped
    assert sorted(O.float().sum(1).tolist()) == pytest.approx(sorted(lin.O_vals.reshape(-1, 8).float().sum(1).tolist()))
    # out of range: huge critical values relative to the codebook step
    big = lin.O_vals.reshape(-1, 8).float() * 1e4
    none = critical_lists(big.half(), lin.O_col, lin.O_row_ptr, N, unit=0.1, code_max=2.0)
    assert none == (None, None, None)
    ok = critical_lists(lin.O_vals, lin.O_col, lin.O_row_ptr, N, unit=0.1, code_max=2.0)
    assert ok[0] is not None and CRIT_ROW_LIMIT > 0
