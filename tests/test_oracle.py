"""The CPU oracle against the fixtures produced by the reference itself."""
import numpy as np
import pytest

import oracle
from tests import util


def test_tables_match_reference_digests():
    ref = util.load_json("tables.json")
    assert util.sha(oracle.e8_raw_points()) == ref["e8_raw_sha256"]
    assert util.sha(oracle.e8_table(1.6)) == ref["e8_r1.6_sha256"]
    assert oracle.e8_table(1.6).shape == (ref["e8_rows"], 8)
    assert util.sha(oracle.d4_raw_codes()) == ref["d4_raw_sha256"]
    assert util.sha(oracle.d4_table(1.75)) == ref["d4_r1.75_sha256"]


def test_e8_table_structure():
    raw = oracle.e8_raw_points()
    n2 = (raw.astype(np.float64) ** 2).sum(1)
    vals, counts = np.unique(n2, return_counts=True)
    assert vals.tolist() == [0, 2, 4, 6, 8, 10, 12]
    assert counts.tolist() == [1, 240, 2160, 6720, 17520, 30240, 8654]
    assert np.abs(raw).max() <= 3.0
    frac = (raw * 2) % 2
    assert ((frac == frac[:, :1]).all(1)).all()          # all-integer or all-half-integer rows


def test_d4_table_structure():
    raw = oracle.d4_raw_codes()
    assert raw.shape == (4, 128, 4)
    s = raw.sum(-1)
    assert (s[0] % 2 == 0).all() and (s[1] % 2 == 0).all()
    assert (s[2] % 2 == 1).all() and (s[3] % 2 == 1).all()
    assert ((raw[0] * 2) % 2 == 0).all() and ((raw[1] * 2) % 2 == 1).all()
    assert len({tuple(r) for r in raw.reshape(-1, 4).tolist()}) == 512


@pytest.mark.parametrize("name", util.CASES)
def test_dequantize_bit_exact(name):
    d = util.load_case(name)
    W = oracle.dequantize_layer(util.case_layer(d), util.oracle_table(d["kind"], d["radius"]))
    assert W.dtype == np.float16
    assert np.array_equal(W.view(np.uint16), d["W16"].view(np.uint16))


@pytest.mark.parametrize("name", util.CASES)
def test_linear_reference(name):
    d = util.load_case(name)
    y = oracle.linear_reference(d["x"], d["W16"], d.get("bias"))
    assert util.max_rel_err(y, d["y"]) < 1e-6


@pytest.mark.parametrize("name", [c for c in util.CASES if "sgroup" not in c])
def test_kernel_formula_agrees_with_reconstruction(name):
    """The un-reconstructed GEMV formula (fp16 table, no fp16 rounding of W) stays
    inside the output gate relative to the reconstruct-then-matmul oracle."""
    d = util.load_case(name)
    tab = util.oracle_table(d["kind"], d["radius"]).astype(np.float16)
    y = oracle.gemv_formula_reference(util.case_layer(d), tab, d["x"])
    assert util.max_rel_err(y, d["y"]) < util.REL_TOL


def test_config1_digest():
    """Full OPT-125m fc1 configuration: inputs re-made from the seed, W16 digest from the reference."""
    from eptq_b200.synthetic import make_layer
    ref = util.load_json("config1.json")
    qd = make_layer(ref["out"], ref["in"], seed=ref["seed"])
    assert util.sha(qd.Q) == ref["Q_sha256"] and util.sha(qd.O) == ref["O_sha256"]
    W = oracle.dequantize_layer(util.qld_arrays(qd), oracle.e8_table(ref["radius"]))
    assert util.sha(W) == ref["W16_sha256"]


def test_csr_from_q():
    d = util.load_case("d4_marker_rows")
    col, ptr = oracle.csr_from_q(d["Q"])
    assert ptr[0] == 0 and ptr[-1] == d["O"].shape[0]
    assert (np.diff(ptr) >= 0).all()
    assert ptr[2] - ptr[1] == d["Q"].shape[1]             # the all-marker row
