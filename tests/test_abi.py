"""The C-ABI library loads and exports every function the header declares (no compute calls)."""
import ctypes
import re
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def declared_functions():
    text = (ROOT / "include" / "eptq_b200.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(eptq_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_entry_points():
    names = declared_functions()
    for must in ("eptq_e8_forward", "eptq_e8d4_forward", "eptq_linear_forward", "eptq_dequantize",
                 "eptq_strerror", "eptq_workspace_bytes", "eptq_abi_version"):
        assert must in names


def test_library_exports_all_declared(built_library):
    lib = ctypes.CDLL(str(built_library))
    for name in declared_functions():
        assert hasattr(lib, name), f"{name} declared in the header but not exported"


def test_binding_covers_all_declared(built_library):
    from eptq_b200 import _lib
    assert sorted(_lib.EXPORTS) == declared_functions()
    lib = _lib.load()
    assert lib.eptq_abi_version() == 3
    assert lib.eptq_strerror(0) == b"ok"
    assert b"workspace" in lib.eptq_strerror(5)
    assert lib.eptq_workspace_bytes(512, 4096, 1) > 0
    assert lib.eptq_workspace_bytes(0, 4096, 1) == 0


def test_argument_checks_need_no_gpu(built_library):
    """Null / shape errors are reported before anything touches the device."""
    from eptq_b200 import _lib
    lib = _lib.load()
    assert lib.eptq_linear_forward(None, None, None, 1, None, 0, None) == 1      # EPTQ_ERR_NULL
    d = _lib.EptqLayer()
    d.quantizer = 7
    assert lib.eptq_dequantize(ctypes.byref(d), None, None) == 4                 # EPTQ_ERR_QUANTIZER
    d.quantizer = 0
    assert lib.eptq_dequantize(ctypes.byref(d), None, None) == 2                 # EPTQ_ERR_SHAPE


def test_prepare_d4_table8_on_host(built_library):
    """Host-only entry point: lattice tables convert exactly, a warped table is refused."""
    import numpy as np
    import oracle
    from eptq_b200 import _lib
    lib = _lib.load()
    tab = np.ascontiguousarray(oracle.d4_table(1.75).reshape(-1))
    out = np.zeros(2048, np.uint8)
    scale = ctypes.c_float(0)
    assert lib.eptq_prepare_d4_table8(tab.ctypes.data, out.ctypes.data, ctypes.addressof(scale)) == 0
    assert abs(scale.value - 0.5 / 1.75) < 1e-6
    # int8 coordinates are twice the raw (half-integer) lattice coordinates
    assert np.array_equal(out.view(np.int8).astype(np.float32) * 0.5, oracle.d4_raw_codes().reshape(-1))
    warped = tab * (1 + 0.05 * np.abs(tab))
    assert lib.eptq_prepare_d4_table8(np.ascontiguousarray(warped).ctypes.data, out.ctypes.data,
                                      ctypes.addressof(scale)) == 7


def test_workspace_sizes_for_long_prefills(built_library):
    """From 1024 tokens on the scratch also holds the reconstructed fp16 weight (16 M N bytes behind the first MiB)."""
    from eptq_b200 import _lib
    lib = _lib.load()
    M, N = 512, 4096
    weight = 8 * M * N * 2
    assert lib.eptq_workspace_bytes(M, N, 1024) == (1 << 20) + weight
    assert lib.eptq_workspace_bytes(M, N, 4096) >= (1 << 20) + weight        # the shape-only bound also covers the SIMT path
    assert lib.eptq_workspace_bytes(M, N, 1023) < (1 << 20) + weight
