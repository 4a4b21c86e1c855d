"""EPTQLinear: ``nn.Linear`` replacement that keeps the weight quantized.

Same constructor, class method, buffers and ``forward`` contract as the
reference module (kernels/linear.py:20-219): buffers ``Q, g, h, O_vals, O_col,
O_row_ptr, bias``; a codebook shared between layers and moved by ``_apply``;
inputs of any leading shape; non-fp16 activations are cast to fp16 and the
result cast back.  Differences, all on purpose:

* one compute path (the C-ABI library), chosen by batch size only -- no Triton,
  no environment switches, no CPU fallback;
* layers with group scales run in the kernel; the reference reconstructs an
  fp16 weight at load time and calls ``F.linear`` (kernels/linear.py:97-120);
* an fp32 copy of the codebook is kept next to the fp16 one, because bit-exact
  reconstruction (``dequantize()`` and the prefill GEMM) needs the table the
  reference's ``dequantize_layer`` reads.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn as nn

import ctypes as C

from .. import _lib
from . import _make_desc, critical_lists, d4_table8, dequantize_layer, linear_forward, linear_forward_group, workspace_for

MARKER = 32767     # int16 value that marks a critical block (index 65535 - 32768)

_table_cache: dict = {}


def _shared_table(codebook: torch.Tensor, dtype: torch.dtype, quantizer_type: str) -> torch.Tensor:
    """One converted copy per (source tensor, dtype): layers of a model share it."""
    key = (codebook.data_ptr(), codebook.device, tuple(codebook.shape), codebook.dtype, dtype,
           codebook._version, quantizer_type)
    hit = _table_cache.get(key)
    if hit is not None:
        return hit
    tab = codebook.detach().to(dtype=dtype)
    tab = tab.reshape(512, 4) if quantizer_type == "e8_d4" else tab
    tab = tab.contiguous()
    if len(_table_cache) > 64:
        from . import clear_derived_caches
        _table_cache.clear()
        clear_derived_caches()                 # their entries are keyed by the tensors dropped here
    _table_cache[key] = tab
    return tab


class EPTQLinear(nn.Module):
    """Quantized linear layer computing ``y = x W^T + bias`` straight from
    ``Q`` (int16 (out/8, in)), the codebook, ``g``, ``h`` and the critical blocks."""

    def __init__(
        self,
        Q: torch.Tensor,
        codebook: torch.Tensor,
        g: torch.Tensor,
        h: torch.Tensor,
        O_vals: torch.Tensor,
        O_col: torch.Tensor,
        O_row_ptr: torch.Tensor,
        bias: Optional[torch.Tensor],
        quantizer_type: str,
        materialized_weight: Optional[torch.Tensor] = None,
        S_group: Optional[torch.Tensor] = None,
        codebook32: Optional[torch.Tensor] = None,
    ):
        super().__init__()
        if quantizer_type not in ("e8_lattice", "e8_d4"):
            raise ValueError(f"unknown quantizer_type {quantizer_type!r}")
        self.in_features = Q.shape[1]
        self.out_features = Q.shape[0] * 8
        self.quantizer_type = quantizer_type

        self.register_buffer("Q", Q.contiguous())
        self.register_buffer("g", g.contiguous())
        self.register_buffer("h", h.contiguous())
        self.register_buffer("O_vals", O_vals.contiguous())
        self.register_buffer("O_col", O_col.contiguous())
        self.register_buffer("O_row_ptr", O_row_ptr.contiguous())
        self.register_buffer("bias", bias.contiguous() if bias is not None else None)
        self.register_buffer("S_group", S_group.contiguous() if S_group is not None else None)
        # Accepted for signature compatibility; this implementation never needs it.
        self.register_buffer("_materialized_weight",
                             materialized_weight.contiguous() if materialized_weight is not None else None)
        self.qb_size = self.out_features // S_group.shape[0] if S_group is not None else 0
        # Critical blocks regrouped by 64 x 128 unit of Q for the streaming GEMV: derived like the CSR tables,
        # not part of the saved state.
        crit = (None, None, None)
        if quantizer_type == "e8_d4" and S_group is None:
            t8 = d4_table8(codebook)                     # None for a warped codebook: no streaming kernel, no range to check
            crit = critical_lists(self.O_vals, self.O_col, self.O_row_ptr, self.in_features,
                                  unit=t8[1] if t8 is not None else None, code_max=float(codebook.abs().max()))
        for name, t in zip(("crit_ptr", "crit_pos", "crit_O"), crit):
            self.register_buffer(name, t, persistent=False)

        # Shared between layers, therefore plain attributes, not buffers.
        self._codebook = codebook
        self._codebook32 = codebook32
        self._desc = None            # cached C-ABI descriptor, dropped whenever the buffers may have moved

    def _apply(self, fn, *args, **kwargs):
        super()._apply(fn, *args, **kwargs)
        self._desc = None
        self._codebook = self._move_shared(self._codebook, fn)
        if self._codebook32 is not None:
            moved = self._move_shared(self._codebook32, fn)
            self._codebook32 = moved if moved.dtype == torch.float32 else self._codebook32.to(moved.device)
        return self

    @staticmethod
    def _move_shared(t: torch.Tensor, fn) -> torch.Tensor:
        key = ("moved", t.data_ptr(), t.device, t.dtype, tuple(t.shape), t._version)
        out = fn(t)
        if out is t:
            return t
        hit = _table_cache.get(key)
        if hit is not None and hit.device == out.device and hit.dtype == out.dtype:
            return hit
        _table_cache[key] = out
        return out

    @classmethod
    def from_quantized_data(cls, quant_data, codebook: torch.Tensor, quantizer_type: str) -> "EPTQLinear":
        """Build the layer from a ``QuantizedLayerData`` and the codebook already
        divided by its radius: (rows, 8) for E8, (4, 128, 4) or (512, 4) for E8-D4."""
        Q = quant_data.Q
        M = Q.shape[0]
        cb16 = _shared_table(codebook, torch.float16, quantizer_type)
        cb32 = _shared_table(codebook, torch.float32, quantizer_type) if codebook.dtype == torch.float32 else None

        # Markers in row-major order: this is the order of the rows of O
        # (algorithms/eptq.py:376-378), so O needs no permutation.
        rows, cols = (Q == MARKER).nonzero(as_tuple=True)
        n_masked = rows.shape[0]
        if quant_data.O.shape[0] != n_masked:
            raise AssertionError(
                f"O shape mismatch: got {quant_data.O.shape[0]} values but found {n_masked} masked positions in Q")
        counts = torch.bincount(rows, minlength=M)
        row_ptr = torch.zeros(M + 1, dtype=torch.int32, device=Q.device)
        row_ptr[1:] = counts.cumsum(0).to(torch.int32)

        return cls(
            Q=Q, codebook=cb16,
            g=quant_data.g.to(torch.float16), h=quant_data.h.to(torch.float16),
            O_vals=quant_data.O.to(torch.float16).reshape(-1, 8),
            O_col=cols.to(torch.int32), O_row_ptr=row_ptr,
            bias=quant_data.bias.to(torch.float16) if quant_data.bias is not None else None,
            quantizer_type=quantizer_type,
            S_group=quant_data.S_group.to(torch.float16) if quant_data.S_group is not None else None,
            codebook32=cb32,
        )

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if not x.is_cuda:
            raise RuntimeError("EPTQLinear runs on CUDA tensors only (there is no CPU path)")
        lead, out_dtype = x.shape[:-1], x.dtype
        x2 = x.reshape(-1, self.in_features)
        if x2.dtype != torch.float16:
            x2 = x2.half()
        if not x2.is_contiguous():
            x2 = x2.contiguous()
        if torch.compiler.is_compiling():
            # traced: go through the registered custom op (one graph node, has a fake implementation)
            y = linear_forward(x2, self.Q, self._codebook, self._codebook32, self.g, self.h,
                               self.O_vals, self.O_col, self.O_row_ptr, self.bias, self.S_group,
                               self.quantizer_type, self.qb_size)
        else:
            y = self._forward_direct(x2)
        if out_dtype != torch.float16:
            y = y.to(out_dtype)
        return y.reshape(*lead, self.out_features)

    def _forward_direct(self, x2: torch.Tensor) -> torch.Tensor:
        """Eager path: cached descriptor, one ctypes call, no dispatcher in between."""
        lib = _lib.load()
        d = self._desc
        if d is None or d.Q != self.Q.data_ptr() or d.h != self.h.data_ptr() or d.g != self.g.data_ptr():
            d = self._desc = self.descriptor()
        B = x2.shape[0]
        y = torch.empty((B, self.out_features), dtype=torch.float16, device=x2.device)
        if B == 0:
            return y
        ws = workspace_for(x2.device, lib.eptq_layer_workspace_bytes(C.byref(d), B))
        if x2.device.index is not None and x2.device.index != torch.cuda.current_device():
            with torch.cuda.device(x2.device):
                st = lib.eptq_linear_forward(C.byref(self._desc), x2.data_ptr(), y.data_ptr(), B, ws.data_ptr(),
                                             ws.numel(), torch.cuda.current_stream(x2.device).cuda_stream)
        else:
            st = lib.eptq_linear_forward(C.byref(self._desc), x2.data_ptr(), y.data_ptr(), B, ws.data_ptr(),
                                         ws.numel(), torch.cuda.current_stream(x2.device).cuda_stream)
        if st != 0:
            _lib.check(st, "eptq linear forward")
        return y

    def dequantize(self) -> torch.Tensor:
        """fp16 (out, in) weight reconstructed on the GPU, bit-identical to the
        reference's ``dequantize_layer`` when the layer was built from an fp32 codebook."""
        if self._codebook32 is None:
            raise RuntimeError("this layer was built from an fp16 codebook; exact reconstruction needs the fp32 table")
        return dequantize_layer(self.Q, self._codebook32, self.g, self.h, self.O_vals, self.O_col,
                                self.O_row_ptr, self.S_group, self.quantizer_type, self.qb_size)

    def descriptor(self):
        """The C-ABI description (struct EptqLayer) of this layer's device buffers."""
        crit = (self.crit_ptr, self.crit_pos, self.crit_O) if self.crit_ptr is not None else None
        return _make_desc(self.quantizer_type, self.Q, self._codebook32, self._codebook, self.g, self.h,
                          self.O_vals, self.O_col, self.O_row_ptr, self.bias, self.S_group, self.qb_size, crit)

    def extra_repr(self) -> str:
        return (f"in={self.in_features}, out={self.out_features}, quantizer={self.quantizer_type}, "
                f"n_masked={self.O_col.shape[0]}")


def forward_group(layers, xs):
    """Apply several independent EPTQLinear layers in one kernel launch: layers[i](xs[i]) for all i.
    Inputs need one common leading shape with at most 16 rows; the layers must share one codebook and have no
    group scales.  Returns the list of outputs.  Meant for q/k/v and gate/up."""
    lead = xs[0].shape[:-1]
    x2 = []
    for lin, x in zip(layers, xs):
        if not x.is_cuda:
            raise RuntimeError("EPTQLinear runs on CUDA tensors only (there is no CPU path)")
        v = x.reshape(-1, lin.in_features)
        v = v if v.dtype == torch.float16 else v.half()
        x2.append(v if v.is_contiguous() else v.contiguous())
    ys = linear_forward_group([lin.descriptor() for lin in layers], x2, [lin.out_features for lin in layers])
    return [y.to(x.dtype).reshape(*lead, lin.out_features) for y, x, lin in zip(ys, xs, layers)]


QuantizedLinear = EPTQLinear
