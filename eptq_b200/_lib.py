"""ctypes binding of ``libeptq_b200.so`` (the C ABI in ``include/eptq_b200.h``).

The library is the only compute path of this package.  If it is missing or a
call fails, a ``RuntimeError`` is raised; nothing falls back to PyTorch.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path
from typing import Optional

LIB_PATH = Path(__file__).resolve().parent / "lib" / "libeptq_b200.so"

EPTQ_E8, EPTQ_E8D4 = 0, 1
QUANTIZER_ID = {"e8_lattice": EPTQ_E8, "e8_d4": EPTQ_E8D4}

# Every symbol the header declares, with (restype, argtypes).
_vp, _i, _sz = C.c_void_p, C.c_int, C.c_size_t
EXPORTS = {
    "eptq_abi_version": (_i, []),
    "eptq_strerror": (C.c_char_p, [_i]),
    "eptq_launch_count": (C.c_uint64, []),
    "eptq_kernel_launch_count": (C.c_uint64, [_i]),
    "eptq_workspace_bytes": (_sz, [_i, _i, _i]),
    "eptq_layer_workspace_bytes": (_sz, [_vp, _i]),
    "eptq_prepare_d4_table8": (_i, [_vp, _vp, _vp]),
    "eptq_e8_forward": (_i, [_vp, _vp, _i, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "eptq_e8d4_forward": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "eptq_forget_codebook": (None, [_vp]),
    "eptq_linear_forward": (_i, [_vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "eptq_dequantize": (_i, [_vp, _vp, _vp]),
    "eptq_group_workspace_bytes": (_sz, [_vp, _i, _i]),
    "eptq_linear_forward_group": (_i, [_vp, _i, _vp, _vp, _i, _vp, _sz, _vp]),
    "eptq_linear_forward_group_fused": (_i, [_vp, _i, _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "eptq_linear_forward_chain": (_i, [_vp, _i, _vp, _vp, _vp, _vp, _i, _vp, _sz, _vp]),
    "eptq_workspace_status": (_i, [_vp, _vp, _vp]),
    "eptq_static_scratch_bytes": (_sz, []),
    "eptq_linear_forward_static_scratch": (_i, [_vp, _vp, _vp, _i, _vp]),
    "eptq_allreduce_data_bytes": (_sz, [_i, _i]),
    "eptq_allreduce_flag_bytes": (_sz, [_i]),
    "eptq_allreduce_push": (_i, [_vp, _vp, _vp, _i, _vp, _vp, _i, _i, _i, _vp]),
    "eptq_allreduce_set_wait_ns": (None, [C.c_uint64]),
    "eptq_lm_head_workspace_bytes": (_sz, [_i]),
    "eptq_lm_head_argmax": (_i, [_vp, _vp, _vp, C.c_float, _vp, _vp, _i, _i, _i, _vp, _sz, _vp]),
    "eptq_add_rmsnorm": (_i, [_vp, _vp, _vp, _vp, _i, _i, C.c_float, _vp]),
    "eptq_silu_mul": (_i, [_vp, _vp, _vp, _sz, _vp]),
    "eptq_rope_append": (_i, [_vp, _vp, _vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, C.c_float, _vp]),
    "eptq_attention_workspace_bytes": (_sz, [_i, _i, _i, _i]),
    "eptq_decode_attention": (_i, [_vp, _vp, _vp, _vp, _vp, _i, _i, _i, _i, _i, _i, C.c_float, _vp, _sz, _vp]),
}


class EptqLayer(C.Structure):
    """struct EptqLayer of include/eptq_b200.h."""
    _fields_ = [
        ("quantizer", C.c_int32), ("M", C.c_int32), ("N", C.c_int32),
        ("n_masked", C.c_int32), ("qb_size", C.c_int32), ("table_rows", C.c_int32),
        ("Q", _vp), ("table32", _vp), ("table16", _vp), ("g", _vp), ("h", _vp),
        ("O_vals", _vp), ("O_col", _vp), ("O_row_ptr", _vp), ("bias", _vp), ("S_group", _vp),
        ("table8", _vp), ("table8_scale", C.c_float), ("h_absmax", C.c_float),
        ("table_packed", _vp), ("table_packed_scale", C.c_float), ("reserved", C.c_int32),
        ("crit_ptr", _vp), ("crit_pos", _vp), ("crit_O", _vp),
    ]


X_PLAIN, X_RMSNORM, X_SILU_MUL = 0, 2, 3
Y_STORE, Y_ADD_RESIDUAL, Y_ROPE, Y_ROPE_TO_CACHE, Y_TO_CACHE = 0, 1, 2, 3, 4


class EptqFusion(C.Structure):
    """struct EptqFusion of include/eptq_b200.h."""
    _fields_ = [
        ("x_op", C.c_int32), ("y_op", C.c_int32), ("norm_eps", C.c_float), ("rope_scaling", C.c_float),
        ("max_len", C.c_int32), ("reserved", C.c_int32),
        ("residual", _vp), ("position", _vp), ("inv_freq", _vp), ("x_aux", _vp),
    ]


_lib: Optional[C.CDLL] = None


def load() -> C.CDLL:
    """Load the library (once) and declare its prototypes."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.exists():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m eptq_b200.build` "
            "(the eptq_b200 kernels have no fallback path)")
    lib = C.CDLL(str(LIB_PATH))
    for name, (res, args) in EXPORTS.items():
        fn = getattr(lib, name)          # AttributeError if the symbol is not exported
        fn.restype, fn.argtypes = res, args
    if lib.eptq_abi_version() != 3:
        raise RuntimeError("libeptq_b200.so has an unexpected ABI version")
    _lib = lib
    return lib


def check(status: int, what: str) -> None:
    if status != 0:
        msg = load().eptq_strerror(status).decode()
        raise RuntimeError(f"{what}: {msg} (eptq status {status})")


KERNEL_GEMV_STREAM, KERNEL_GEMV_GROUP, KERNEL_GEMV_MMA, KERNEL_GEMV_SIMT, KERNEL_GEMM, KERNEL_OTHER = range(6)


def kernel_launch_count(kernel: int) -> int:
    return int(load().eptq_kernel_launch_count(kernel))


def launch_count() -> int:
    return int(load().eptq_launch_count())
