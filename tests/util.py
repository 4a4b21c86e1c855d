"""Shared helpers of the test-suite: golden cases, oracle adapters, error metric."""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import numpy as np
import torch

import oracle
from eptq_b200.config import QuantizedLayerData

GOLDEN = Path(__file__).resolve().parent / "golden"
CASES = sorted(p.stem[len("case_"):] for p in GOLDEN.glob("case_*.npz"))

# Gate on layer outputs: max_i |y_i - yref_i| / max_i |yref_i| <= 2e-3.
REL_TOL = 2e-3


def sha(a) -> str:
    if isinstance(a, torch.Tensor):
        a = a.detach().cpu().contiguous().numpy()
    return hashlib.sha256(np.ascontiguousarray(a).tobytes()).hexdigest()


def load_json(name: str) -> dict:
    return json.loads((GOLDEN / name).read_text())


def load_case(name: str) -> dict:
    z = np.load(GOLDEN / f"case_{name}.npz")
    d = {k: z[k] for k in z.files}
    d["kind"] = str(d["kind"])
    d["radius"] = float(d["radius"])
    return d


def oracle_table(kind: str, radius: float) -> np.ndarray:
    return oracle.e8_table(radius) if kind == "e8_lattice" else oracle.d4_table(radius)


def case_layer(d: dict) -> oracle.LayerArrays:
    return oracle.LayerArrays(Q=d["Q"], g=d["g"], h=d["h"], O=d["O"], bias=d.get("bias"), S_group=d.get("S_group"))


def case_qld(d: dict) -> QuantizedLayerData:
    t = lambda k: torch.from_numpy(d[k].copy()) if k in d else None   # noqa: E731
    return QuantizedLayerData(Q=t("Q"), g=t("g"), h=t("h"), O=t("O"), bias=t("bias"), S_group=t("S_group"))


def qld_arrays(qd: QuantizedLayerData) -> oracle.LayerArrays:
    n = lambda t: None if t is None else t.detach().cpu().numpy()      # noqa: E731
    return oracle.LayerArrays(Q=n(qd.Q), g=n(qd.g), h=n(qd.h), O=n(qd.O), bias=n(qd.bias), S_group=n(qd.S_group))


def max_rel_err(y, y_ref) -> float:
    y = np.asarray(y, dtype=np.float64)
    y_ref = np.asarray(y_ref, dtype=np.float64)
    return float(np.abs(y - y_ref).max() / max(np.abs(y_ref).max(), 1e-30))
