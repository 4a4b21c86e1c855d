"""Op-level API of the quantized-linear path.

``e8_forward`` and ``e8d4_forward`` keep the reference's signatures
(kernels/__init__.py:50-84, csrc/eptq_kernels.h:15-41) and are registered as
``torch.library.custom_op`` with fake implementations, so ``torch.compile`` and
CUDA-graph capture see them as single ops, as in the reference
(kernels/__init__.py:46-91).  They are registered under the namespace
``eptq_b200`` so that the reference package can be imported next to this one.

``linear_forward`` takes the whole layer (group scales included) and
``dequantize_layer`` reconstructs the fp16 weight on the GPU, bit-for-bit the
reference's ``dequantize_layer`` (algorithms/eptq.py:406-471).

Inputs must be CUDA tensors; a CPU tensor raises -- there is no CPU path.
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch

from .. import _lib

__all__ = ["e8_forward", "e8d4_forward", "linear_forward", "linear_forward_group", "linear_forward_chain",
           "dequantize_layer", "workspace_for", "workspace_status", "workspace_status_all"]

_workspaces: Dict[Tuple[int, int], torch.Tensor] = {}


def workspace_for(device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch for (device, current stream), grown on demand.

    Calls ordered on one stream share it; the kernels leave it zeroed where they
    need zeros.  Growing allocates, so size it before capturing a CUDA graph."""
    stream = torch.cuda.current_stream(device)
    key = (device.index if device.index is not None else torch.cuda.current_device(), stream.cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _require_cuda(**tensors) -> None:
    for name, t in tensors.items():
        if t is not None and not t.is_cuda:
            raise RuntimeError(f"eptq_b200: `{name}` must be a CUDA tensor (no CPU path exists)")


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None or t.numel() == 0 else t.data_ptr()


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _check_common(Q, g, h, x):
    if Q.dtype != torch.int16 or not Q.is_contiguous():
        raise RuntimeError("Q must be a contiguous CUDA int16 tensor")
    if x.dtype != torch.float16 or not x.is_contiguous():
        raise RuntimeError("x must be a contiguous CUDA fp16 tensor")
    if x.dim() != 2 or x.shape[1] != Q.shape[1]:
        raise RuntimeError(f"x must have shape (B, {Q.shape[1]})")
    if g.dtype != torch.float16 or h.dtype != torch.float16:
        raise RuntimeError("g and h must be fp16")


def _forward_impl(kind: str, Q, table, g, h, x, O_vals, O_col, O_row_ptr, bias) -> torch.Tensor:
    _require_cuda(Q=Q, codebook=table, g=g, h=h, x=x, O_vals=O_vals, O_col=O_col, O_row_ptr=O_row_ptr)
    _check_common(Q, g, h, x)
    if table.dtype != torch.float16 or not table.is_contiguous():
        raise RuntimeError("codebook must be a contiguous fp16 tensor")
    lib = _lib.load()
    M, N = Q.shape
    B = x.shape[0]
    y = torch.empty((B, M * 8), dtype=torch.float16, device=x.device)
    if B == 0:
        return y
    nbytes = lib.eptq_workspace_bytes(M, N, B)
    ws = workspace_for(x.device, nbytes)
    with torch.cuda.device(x.device):
        if kind == "e8_lattice":
            # through the descriptor, so that the packed table (made once per codebook tensor) reaches the
            # persistent kernel; eptq_e8_forward itself only knows the fp16 table
            desc = _make_desc("e8_lattice", Q, None, table, g, h, O_vals, O_col, O_row_ptr,
                              None if bias is None or bias.numel() == 0 else bias, None, 0)
            st = lib.eptq_linear_forward(C.byref(desc), x.data_ptr(), y.data_ptr(), B,
                                         ws.data_ptr(), ws.numel(), _stream(x.device))
        else:
            if table.numel() != 2048:
                raise RuntimeError("E8-D4 codes must hold 512 x 4 values")
            desc = _make_desc("e8_d4", Q, None, table, g, h, O_vals, O_col, O_row_ptr,
                              None if bias is None or bias.numel() == 0 else bias, None, 0)
            st = lib.eptq_linear_forward(C.byref(desc), x.data_ptr(), y.data_ptr(), B,
                                         ws.data_ptr(), ws.numel(), _stream(x.device))
    _lib.check(st, f"eptq {kind} forward")
    return y


@torch.library.custom_op("eptq_b200::e8_forward", mutates_args=())
def e8_forward(Q: torch.Tensor, codebook: torch.Tensor, g: torch.Tensor, h: torch.Tensor, x: torch.Tensor,
               O_vals: torch.Tensor, O_col: torch.Tensor, O_row_ptr: torch.Tensor,
               bias: torch.Tensor) -> torch.Tensor:
    """E8 fused dequantise + GEMV.  Arguments as the reference's ``e8_forward``
    (csrc/eptq_kernels.h:4-25); an empty ``bias`` tensor means no bias.  Returns a
    new (B, 8M) fp16 tensor on x's device."""
    return _forward_impl("e8_lattice", Q, codebook, g, h, x, O_vals, O_col, O_row_ptr, bias)


@e8_forward.register_fake
def _(Q, codebook, g, h, x, O_vals, O_col, O_row_ptr, bias):
    return x.new_empty(x.shape[0], Q.shape[0] * 8, dtype=torch.float16)


@torch.library.custom_op("eptq_b200::e8d4_forward", mutates_args=())
def e8d4_forward(Q: torch.Tensor, codes: torch.Tensor, g: torch.Tensor, h: torch.Tensor, x: torch.Tensor,
                 O_vals: torch.Tensor, O_col: torch.Tensor, O_row_ptr: torch.Tensor,
                 bias: torch.Tensor) -> torch.Tensor:
    """E8-D4 fused dequantise + GEMV.  ``codes`` is the fp16 (512, 4) table
    (csrc/eptq_kernels.h:27-41)."""
    return _forward_impl("e8_d4", Q, codes, g, h, x, O_vals, O_col, O_row_ptr, bias)


@e8d4_forward.register_fake
def _(Q, codes, g, h, x, O_vals, O_col, O_row_ptr, bias):
    return x.new_empty(x.shape[0], Q.shape[0] * 8, dtype=torch.float16)


_table8_cache: Dict[tuple, Optional[Tuple[torch.Tensor, float]]] = {}
# Derived values are cached by the address of their source tensor; the cache keeps that tensor alive, so that the
# allocator cannot hand the address to another tensor while an entry is valid.  clear_derived_caches() drops all.
_cache_sources: Dict[tuple, torch.Tensor] = {}


def clear_derived_caches() -> None:
    """Forget every table / scale derived from a tensor (int8 and packed tables, max |h|)."""
    _table8_cache.clear()
    _packed_cache.clear()
    _absmax_cache.clear()
    _cache_sources.clear()



def d4_table8(table: torch.Tensor):
    """(host int8 (2048,) numpy array, scale) with the E8-D4 table expressed as
    scale * integer lattice coordinates, or None if the table is not such a multiple
    (a radially warped codebook).  Prepared on the host once per table tensor; the
    library copies it into the kernel parameters at each launch."""
    key = (table.data_ptr(), table.device, table.dtype, table._version)
    if key in _table8_cache:
        return _table8_cache[key]
    import numpy as np
    host = np.ascontiguousarray(table.detach().float().cpu().numpy().reshape(-1))
    res = None
    if host.size == 2048:
        out = np.zeros(2048, dtype=np.uint8)
        scale = C.c_float(0.0)
        st = _lib.load().eptq_prepare_d4_table8(host.ctypes.data, out.ctypes.data, C.addressof(scale))
        if st == 0:
            res = (out.view(np.int8), float(scale.value))
    if len(_table8_cache) > 64:
        _table8_cache.clear()
    _table8_cache[key] = res
    _cache_sources[("t8",) + key] = table          # the keyed tensor stays alive: its address cannot be reused
    return res


_packed_cache: Dict[tuple, Optional[Tuple[torch.Tensor, float]]] = {}
_E8_FIELD = (0, 4, 1, 5, 2, 6, 3, 7)      # 4-bit field index of dimension d; field f sits at bit 2 + 4 f


def pack_e8_table(table: torch.Tensor) -> Optional[Tuple[torch.Tensor, float]]:
    """(int32 (65536,) tensor on the table's device, scale) with the E8 table written as
    scale * half-integer lattice coordinates, one packed word per entry (layout: `table_packed` in
    include/eptq_b200.h); entries past the table's rows decode to the zero vector.  None if the table is
    not such a multiple (a radially warped codebook) or has coordinates outside [-3, 3]."""
    t = table.detach().float()
    if t.dim() != 2 or t.shape[1] != 8 or t.shape[0] > 65535 or t.shape[0] == 0:
        return None
    nz = t.abs()[t != 0]
    if nz.numel() == 0:
        return None
    scale = 2.0 * float(nz.min())
    twice = torch.round(t * (2.0 / scale))
    # 1e-3: a table already rounded to fp16 still packs (its entries are within 5e-4 of the lattice)
    if float((twice * (scale / 2.0) - t).abs().max()) > 1e-3 * scale or float(twice.abs().max()) > 6:
        return None
    n = (twice + 6).to(torch.int64)                                         # 0..12
    full = torch.full((65536, 8), 6, dtype=torch.int64, device=t.device)
    full[: t.shape[0]] = n
    word = torch.zeros(65536, dtype=torch.int64, device=t.device)
    for d, f in enumerate(_E8_FIELD):
        word |= full[:, d] << (2 + 4 * f)
    word = (word & 0xFFFFFFFF) | (word >> 32)                               # the last field wraps around
    word = torch.where(word >= 2 ** 31, word - 2 ** 32, word).to(torch.int32)
    return word.contiguous(), scale


def unpack_e8_table(word: torch.Tensor, scale: float) -> torch.Tensor:
    """Inverse of pack_e8_table (fp32 (65536, 8)); what the kernel's decode computes."""
    w = word.to(torch.int64) & 0xFFFFFFFF
    w = w | ((w & 0x3) << 32)
    cols = [((w >> (2 + 4 * f)) & 0xF).float() for f in _E8_FIELD]
    return (torch.stack(cols, dim=1) - 6.0) * (scale / 2.0)


def e8_packed(table: torch.Tensor) -> Optional[Tuple[torch.Tensor, float]]:
    """pack_e8_table cached per table tensor (one host sync the first time)."""
    key = (table.data_ptr(), table.device, table.dtype, tuple(table.shape), table._version)
    if key not in _packed_cache:
        if len(_packed_cache) > 64:
            _packed_cache.clear()
        _packed_cache[key] = pack_e8_table(table)
        _cache_sources[("packed",) + key] = table
    return _packed_cache[key]


_absmax_cache: Dict[tuple, float] = {}


def h_absmax(h: torch.Tensor) -> float:
    """max |h| of a column-scale vector, computed once per tensor (one device sync) and cached.
    The persistent GEMV derives its activation scale from it."""
    key = (h.data_ptr(), h.device, h.numel(), h._version)
    v = _absmax_cache.get(key)
    if v is None:
        v = float(h.abs().max().item()) if h.numel() else 0.0
        if len(_absmax_cache) > 4096:
            for k in [k for k in _cache_sources if k[0] == "absmax"]:
                del _cache_sources[k]
            _absmax_cache.clear()
        _absmax_cache[key] = v
        _cache_sources[("absmax",) + key] = h
    return v


CRIT_ROW_LIMIT = 3900.0


def critical_lists(O_vals: torch.Tensor, O_col: torch.Tensor, O_row_ptr: torch.Tensor, N: int,
                   unit: Optional[float] = None, code_max: float = 0.0):
    """The critical blocks regrouped by the 64-row x 128-column unit of Q they fall into (fields crit_ptr,
    crit_pos, crit_O of struct EptqLayer), from the CSR side tables: (int32 (units+1), int32 (n) bit pattern of
    uint32 (row % 64) << 16 | col, fp16 (n, 8)).

    The streaming kernel sums the corrections of a row in 32-bit fixed point; with ``unit`` (the codebook's
    coordinate step) given, a layer whose rows could exceed that range -- sum over a row's critical blocks of
    (|O| + code_max) / unit >= CRIT_ROW_LIMIT in some dimension -- gets (None, None, None) and runs from the CSR
    tables instead."""
    M = O_row_ptr.shape[0] - 1
    dev = O_col.device
    counts = (O_row_ptr[1:] - O_row_ptr[:-1]).to(torch.int64)
    rows = torch.repeat_interleave(torch.arange(M, device=dev), counts)
    if unit is not None and rows.numel() > 0:
        mag = (O_vals.reshape(-1, 8).float().abs() + code_max) / unit
        per_row = torch.zeros(M, 8, device=dev).index_add_(0, rows, mag)
        if float(per_row.max()) >= CRIT_ROW_LIMIT:
            return None, None, None
    cols = O_col.to(torch.int64)
    cc = (N + 127) // 128
    units = ((M + 63) // 64) * cc
    unit = (rows // 64) * cc + cols // 128
    order = torch.argsort(unit, stable=True)
    ptr = torch.zeros(units + 1, dtype=torch.int32, device=dev)
    ptr[1:] = torch.bincount(unit, minlength=units).cumsum(0).to(torch.int32)
    pos = (((rows % 64) << 16) | cols)[order].to(torch.int32)
    return ptr.contiguous(), pos.contiguous(), O_vals.reshape(-1, 8)[order].contiguous()


def _make_desc(quantizer_type: str, Q, table32, table16, g, h, O_vals, O_col, O_row_ptr, bias, S_group,
               qb_size: int, crit=None) -> _lib.EptqLayer:
    d = _lib.EptqLayer()
    d.quantizer = _lib.QUANTIZER_ID[quantizer_type]
    d.M, d.N = Q.shape
    d.n_masked = int(O_col.shape[0]) if O_col is not None else 0
    d.qb_size = int(qb_size) if S_group is not None else 0
    tab = table16 if table16 is not None else table32
    d.table_rows = 512 if quantizer_type == "e8_d4" else int(tab.shape[0])
    d.Q = Q.data_ptr()
    d.table32 = _ptr(table32)
    d.table16 = _ptr(table16)
    d.g, d.h = g.data_ptr(), h.data_ptr()
    d.O_vals, d.O_col, d.O_row_ptr = _ptr(O_vals), _ptr(O_col), O_row_ptr.data_ptr()
    d.bias, d.S_group = _ptr(bias), _ptr(S_group)
    d.table8, d.table8_scale = None, 0.0
    d.h_absmax = h_absmax(h) if Q.is_cuda else 0.0
    d.table_packed, d.table_packed_scale = None, 0.0
    d.crit_ptr = d.crit_pos = d.crit_O = None
    if crit is not None:
        d.crit_ptr, d.crit_pos, d.crit_O = crit[0].data_ptr(), _ptr(crit[1]), _ptr(crit[2])
    if quantizer_type == "e8_lattice" and Q.is_cuda:
        packed = e8_packed(table32 if table32 is not None else table16)
        if packed is not None:
            d._keep = packed[0]                  # keep the device table alive as long as the descriptor
            d.table_packed, d.table_packed_scale = packed[0].data_ptr(), packed[1]
    if quantizer_type == "e8_d4":
        t8 = d4_table8(table32 if table32 is not None else table16)
        if t8 is not None:
            d._keep = t8[0]                      # keep the host table alive as long as the descriptor
            d.table8, d.table8_scale = t8[0].ctypes.data, t8[1]
    return d


@torch.library.custom_op("eptq_b200::linear_forward", mutates_args=())
def linear_forward(x: torch.Tensor, Q: torch.Tensor, table16: torch.Tensor, table32: Optional[torch.Tensor],
                   g: torch.Tensor, h: torch.Tensor, O_vals: torch.Tensor, O_col: torch.Tensor,
                   O_row_ptr: torch.Tensor, bias: Optional[torch.Tensor], S_group: Optional[torch.Tensor],
                   quantizer_type: str, qb_size: int) -> torch.Tensor:
    """Layer forward from the full layer description: (B, in) fp16 -> (B, out) fp16,
    group scales applied in the kernel."""
    _require_cuda(Q=Q, table16=table16, g=g, h=h, x=x, O_row_ptr=O_row_ptr)
    _check_common(Q, g, h, x)
    lib = _lib.load()
    M, N = Q.shape
    B = x.shape[0]
    y = torch.empty((B, M * 8), dtype=torch.float16, device=x.device)
    if B == 0:
        return y
    desc = _make_desc(quantizer_type, Q, table32, table16, g, h, O_vals, O_col, O_row_ptr, bias, S_group, qb_size)
    ws = workspace_for(x.device, lib.eptq_layer_workspace_bytes(C.byref(desc), B))
    with torch.cuda.device(x.device):
        st = lib.eptq_linear_forward(C.byref(desc), x.data_ptr(), y.data_ptr(), B,
                                     ws.data_ptr(), ws.numel(), _stream(x.device))
    _lib.check(st, "eptq linear forward")
    return y


@linear_forward.register_fake
def _(x, Q, table16, table32, g, h, O_vals, O_col, O_row_ptr, bias, S_group, quantizer_type, qb_size):
    return x.new_empty(x.shape[0], Q.shape[0] * 8, dtype=torch.float16)


def linear_forward_group(descs, xs, out_features, workspace: Optional[torch.Tensor] = None,
                         fusions=None, ys=None):
    """Several independent layers in one launch (eptq_linear_forward_group[_fused]).  `descs` are EptqLayer
    descriptors (see EPTQLinear.descriptor), `xs` contiguous fp16 CUDA tensors (B, in_i) with one B;
    returns the list of (B, out_i) fp16 outputs.  `fusions`: optional list of _lib.EptqFusion, one per
    layer; `ys`: optional list of output tensors to write (None entries are allocated) -- a residual
    stream updated in place, or a key/value cache.  Raises if the group is not eligible."""
    lib = _lib.load()
    n = len(descs)
    B = xs[0].shape[0]
    dev = xs[0].device
    ys = list(ys) if ys is not None else [None] * n
    for i, o in enumerate(out_features):
        if ys[i] is None:
            ys[i] = torch.empty((B, o), dtype=torch.float16, device=dev)
    arr = (_lib.EptqLayer * n)(*descs)
    need = lib.eptq_group_workspace_bytes(arr, n, B)
    if need == 0:
        raise RuntimeError("eptq_b200: this set of layers cannot run as one group launch")
    ws = workspace if workspace is not None else workspace_for(dev, need)
    xp = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    with torch.cuda.device(dev):
        if fusions is None:
            st = lib.eptq_linear_forward_group(arr, n, xp, yp, B, ws.data_ptr(), ws.numel(), _stream(dev))
        else:
            fz = (_lib.EptqFusion * n)(*fusions)
            st = lib.eptq_linear_forward_group_fused(arr, n, fz, xp, yp, B, ws.data_ptr(), ws.numel(), _stream(dev))
    _lib.check(st, "eptq group forward")
    return ys


def linear_forward_chain(descs, phases, xs, out_features, fusions, ys=None, workspace: Optional[torch.Tensor] = None):
    """Layers in dependent phases in ONE launch (eptq_linear_forward_chain): a layer of phase k+1 may read
    (as x, x_aux or residual) what a layer of phase k wrote.  Arguments as linear_forward_group plus
    `phases`, the phase of each layer (non-decreasing from 0).  Batch 1, E8-D4 layers of the streaming
    kernel; raises otherwise."""
    lib = _lib.load()
    n = len(descs)
    B = xs[0].shape[0]
    dev = xs[0].device
    ys = list(ys) if ys is not None else [None] * n
    for i, o in enumerate(out_features):
        if ys[i] is None:
            ys[i] = torch.empty((B, o), dtype=torch.float16, device=dev)
    arr = (_lib.EptqLayer * n)(*descs)
    ws = workspace if workspace is not None else workspace_for(dev, 1 << 20)
    xp = (C.c_void_p * n)(*[x.data_ptr() for x in xs])
    yp = (C.c_void_p * n)(*[y.data_ptr() for y in ys])
    ph = (C.c_int * n)(*[int(v) for v in phases])
    fz = (_lib.EptqFusion * n)(*fusions)
    with torch.cuda.device(dev):
        st = lib.eptq_linear_forward_chain(arr, n, fz, ph, xp, yp, B, ws.data_ptr(), ws.numel(), _stream(dev))
    _lib.check(st, "eptq chained forward")
    return ys


def workspace_status(workspace: Optional[torch.Tensor] = None, device=None) -> int:
    """Read and clear the status word of a scratch buffer (eptq_workspace_status): 0, or the code a kernel
    left when one of its bounded waits ran out.  Synchronises the current stream."""
    lib = _lib.load()
    dev = workspace.device if workspace is not None else torch.device(device if device is not None else "cuda")
    ws = workspace if workspace is not None else workspace_for(dev, 1 << 20)
    out = C.c_int(0)
    with torch.cuda.device(dev):
        _lib.check(lib.eptq_workspace_status(ws.data_ptr(), C.addressof(out), _stream(dev)), "eptq workspace status")
    return int(out.value)


def workspace_status_all(device) -> int:
    """workspace_status of every scratch buffer this module made on `device` (one per stream that ran the
    kernels, e.g. the stream a CUDA graph was captured on): the first non-zero code, or 0."""
    dev = torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()
    first = 0
    for (d, _stream_id), ws in list(_workspaces.items()):
        if d == index:
            code = workspace_status(ws)
            first = first or code
    return first


def dequantize_layer(Q: torch.Tensor, table32: torch.Tensor, g: torch.Tensor, h: torch.Tensor,
                     O_vals: torch.Tensor, O_col: torch.Tensor, O_row_ptr: torch.Tensor,
                     S_group: Optional[torch.Tensor], quantizer_type: str, qb_size: int = 0) -> torch.Tensor:
    """fp16 (out, in) weight, bit-identical to the reference's ``dequantize_layer``
    (algorithms/eptq.py:406-471) given the same fp32 table."""
    _require_cuda(Q=Q, table32=table32, g=g, h=h, O_row_ptr=O_row_ptr)
    if table32.dtype != torch.float32 or not table32.is_contiguous():
        raise RuntimeError("table32 must be a contiguous fp32 tensor")
    lib = _lib.load()
    M, N = Q.shape
    W = torch.empty((M * 8, N), dtype=torch.float16, device=Q.device)
    desc = _make_desc(quantizer_type, Q, table32, None, g, h, O_vals, O_col, O_row_ptr, None, S_group, qb_size)
    with torch.cuda.device(Q.device):
        st = lib.eptq_dequantize(C.byref(desc), W.data_ptr(), _stream(Q.device))
    _lib.check(st, "eptq dequantize")
    return W
