"""Regenerates the golden fixtures in this directory from the reference itself.

Needs a checkout of the reference (kmudmlab/eptq): pass its path in the
environment variable EPTQ_REFERENCE.  It is imported as package ``eptq``
through a temporary symlink and run on the CPU.  What is stored:

  tables.json          sha256 of the reference's fp32 codebooks (raw and divided)
  case_*.npz           small layers: inputs, the reference's ``dequantize_layer``
                       output W16 (fp16 bits) and y = x.float() @ W16.float().T (+bias)
  config1.json         sha256 of W16 for the full OPT-125m fc1 configuration
                       (3072x768, E8 r=1.6, seed 42) built by eptq_b200.synthetic

Usage:  EPTQ_REFERENCE=<path to the reference checkout> python tests/golden/make_golden.py
"""
import hashlib
import json
import os
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
REPO = HERE.parent.parent
sys.path.insert(0, str(REPO))

if "EPTQ_REFERENCE" not in os.environ:
    raise SystemExit("set EPTQ_REFERENCE to the path of the reference checkout")
ref_root = Path(os.environ["EPTQ_REFERENCE"])
tmp = tempfile.mkdtemp()
os.symlink(ref_root, Path(tmp) / "eptq")
sys.path.insert(0, tmp)

from eptq.algorithms.eptq import dequantize_layer            # noqa: E402
from eptq.config import QuantizedLayerData as RefQLD         # noqa: E402
from eptq.quantizers import E8D4Quantizer, E8LatticeQuantizer  # noqa: E402

from eptq_b200.synthetic import make_activations, make_layer  # noqa: E402


def sha(t) -> str:
    a = t.detach().cpu().contiguous().numpy() if isinstance(t, torch.Tensor) else np.ascontiguousarray(t)
    return hashlib.sha256(a.tobytes()).hexdigest()


e8 = E8LatticeQuantizer(device="cpu", radius=1.6)
e8.remove_last()
d4 = E8D4Quantizer(device="cpu", radius=1.75)

tables = {
    "e8_raw_sha256": sha(e8._raw_points), "e8_r1.6_sha256": sha(e8.points),
    "e8_rows": int(e8.points.shape[0]),
    "d4_raw_sha256": sha(d4._raw_codes), "d4_r1.75_sha256": sha(d4.codes),
    "torch": torch.__version__,
}
(HERE / "tables.json").write_text(json.dumps(tables, indent=1) + "\n")


def ref_qld(qd, chosen_r=None):
    return RefQLD(Q=qd.Q, g=qd.g, h=qd.h, O=qd.O, bias=qd.bias, chosen_r=chosen_r, S_group=qd.S_group)


def emit(name, qd, quantizer, kind, radius, chosen_r=None, batch=3):
    W16 = dequantize_layer(ref_qld(qd, chosen_r), quantizer)
    assert W16.dtype == torch.float16
    x = make_activations(batch, qd.Q.shape[1], seed=7)
    y = x.float() @ W16.float().T
    if qd.bias is not None:
        y = y + qd.bias.float()
    arrs = dict(Q=qd.Q.numpy(), g=qd.g.numpy(), h=qd.h.numpy(), O=qd.O.numpy(), x=x.numpy(),
                W16=W16.numpy(), y=y.numpy(), kind=np.array(kind),
                radius=np.array(chosen_r if chosen_r is not None else radius, dtype=np.float64))
    if qd.bias is not None:
        arrs["bias"] = qd.bias.numpy()
    if qd.S_group is not None:
        arrs["S_group"] = qd.S_group.numpy()
    np.savez_compressed(HERE / f"case_{name}.npz", **arrs)
    print(name, tuple(W16.shape), "markers", qd.O.shape[0])


emit("e8_basic", make_layer(64, 96, seed=1, outlier_frac=0.01), e8, "e8_lattice", 1.6)
emit("e8_bias_chosen_r", make_layer(32, 64, seed=2, outlier_frac=0.02, bias=True), e8, "e8_lattice", 1.6, chosen_r=1.45)
emit("e8_sgroup", make_layer(128, 40, seed=3, outlier_frac=0.01, qb_size=64), e8, "e8_lattice", 1.6)
emit("d4_basic", make_layer(64, 128, seed=4, outlier_frac=0.01), d4, "e8_d4", 1.75)
emit("d4_sgroup_bias", make_layer(256, 64, seed=5, outlier_frac=0.01, bias=True, qb_size=128), d4, "e8_d4", 1.75)
emit("d4_no_markers", make_layer(16, 40, seed=6, outlier_frac=0.0), d4, "e8_d4", 1.75)
emit("d4_chosen_r", make_layer(48, 72, seed=8, outlier_frac=0.01), d4, "e8_d4", 1.75, chosen_r=1.9)

# A row that is all markers, markers at row start and row end, ragged N.
qd = make_layer(24, 19, seed=9, outlier_frac=0.0)
idx = qd.Q.clone()
idx[1, :] = 32767
idx[0, 0] = 32767
idx[2, -1] = 32767
n = int((idx == 32767).sum())
gen = torch.Generator().manual_seed(10)
qd.Q, qd.O = idx, torch.randn((n, 8), generator=gen).to(torch.float16)
emit("d4_marker_rows", qd, d4, "e8_d4", 1.75)
qd2 = make_layer(24, 19, seed=11, outlier_frac=0.0)
qd2.Q, qd2.O = idx.clone(), qd.O.clone()
emit("e8_marker_rows", qd2, e8, "e8_lattice", 1.6)

# Full configuration 1 (OPT-125m fc1): only a digest, the inputs are re-made from the seed.
qd = make_layer(3072, 768, seed=42)
W16 = dequantize_layer(ref_qld(qd), e8)
x = make_activations(1, 768, seed=42)
y = x.float() @ W16.float().T
(HERE / "config1.json").write_text(json.dumps({
    "out": 3072, "in": 768, "seed": 42, "kind": "e8_lattice", "radius": 1.6,
    "Q_sha256": sha(qd.Q), "O_sha256": sha(qd.O), "g_sha256": sha(qd.g), "h_sha256": sha(qd.h),
    "W16_sha256": sha(W16), "n_markers": int(qd.O.shape[0]),
    "y_abs_max": float(y.abs().max()), "y_first8": [float(v) for v in y[0, :8]],
}, indent=1) + "\n")

# Llama-2-7B q_proj shape with E8-D4 (configuration 2): digest only.
qd = make_layer(4096, 4096, seed=42)
W16 = dequantize_layer(ref_qld(qd), d4)
(HERE / "config2_qproj.json").write_text(json.dumps({
    "out": 4096, "in": 4096, "seed": 42, "kind": "e8_d4", "radius": 1.75,
    "Q_sha256": sha(qd.Q), "W16_sha256": sha(W16), "n_markers": int(qd.O.shape[0]),
}, indent=1) + "\n")
print("done")
