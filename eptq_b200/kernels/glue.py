"""Python face of the decode-step glue kernels (eptq_add_rmsnorm, eptq_silu_mul, eptq_rope_append,
eptq_decode_attention): fp16 CUDA tensors in, raw pointers through the C ABI, launches on the current
stream.  No fallback: a CPU tensor or a missing library raises."""
from __future__ import annotations

from typing import Dict, Optional

import torch

from .. import _lib


def _stream(dev: torch.device) -> int:
    return torch.cuda.current_stream(dev).cuda_stream


def _need(**tensors) -> None:
    for name, t in tensors.items():
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError(f"eptq_b200: `{name}` must be a CUDA tensor (there is no CPU path)")
        if not t.is_contiguous():
            raise RuntimeError(f"eptq_b200: `{name}` must be contiguous")


def add_rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float, delta: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x (rows, H) fp16 is updated in place with `delta` when given; returns the normalised rows."""
    _need(x=x, weight=weight, delta=delta, out=out)
    if x.dtype != torch.float16 or weight.dtype != torch.float16:
        raise RuntimeError("eptq_b200: add_rmsnorm takes fp16 tensors")
    rows, H = x.shape
    out = torch.empty_like(x) if out is None else out
    st = _lib.load().eptq_add_rmsnorm(x.data_ptr(), None if delta is None else delta.data_ptr(), weight.data_ptr(),
                                      out.data_ptr(), rows, H, float(eps), _stream(x.device))
    _lib.check(st, "eptq add_rmsnorm")
    return out


def silu_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    _need(gate=gate, up=up)
    out = torch.empty_like(gate)
    st = _lib.load().eptq_silu_mul(gate.data_ptr(), up.data_ptr(), out.data_ptr(), gate.numel(), _stream(gate.device))
    _lib.check(st, "eptq silu_mul")
    return out


def rope_append(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor,
                positions: torch.Tensor, inv_freq: torch.Tensor, batch: int, scaling: float = 1.0) -> None:
    """q (B*T, nh*hd) rotated in place; k, v (B*T, nkv*hd) appended to the caches (B, nkv, max_len, hd)."""
    _need(q=q, k=k, v=v, k_cache=k_cache, v_cache=v_cache, positions=positions, inv_freq=inv_freq)
    B, nkv, max_len, hd = k_cache.shape
    T = q.shape[0] // batch
    if positions.dtype != torch.int64 or positions.numel() != T or inv_freq.dtype != torch.float32:
        raise RuntimeError("eptq_b200: rope_append needs int64 positions (T,) and fp32 inv_freq")
    st = _lib.load().eptq_rope_append(q.data_ptr(), k.data_ptr(), v.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                                      positions.data_ptr(), inv_freq.data_ptr(), batch, T, q.shape[1] // hd, nkv, hd,
                                      max_len, float(scaling), _stream(q.device))
    _lib.check(st, "eptq rope_append")


_att_ws: Dict[tuple, torch.Tensor] = {}


def decode_attention(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, positions: torch.Tensor,
                     batch: int, scale: Optional[float] = None) -> torch.Tensor:
    """Attention of the rows of q (B*T, nh*hd) over cache positions 0..positions[t]."""
    _need(q=q, k_cache=k_cache, v_cache=v_cache, positions=positions)
    lib = _lib.load()
    B, nkv, max_len, hd = k_cache.shape
    rows = q.shape[0]
    nh = q.shape[1] // hd
    need = lib.eptq_attention_workspace_bytes(rows, nh, hd, max_len)
    key = (q.device, torch.cuda.current_stream(q.device).cuda_stream)
    ws = _att_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _att_ws[key] = torch.zeros(max(need, 1 << 20), dtype=torch.uint8, device=q.device)
    out = torch.empty_like(q)
    st = lib.eptq_decode_attention(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), positions.data_ptr(),
                                   out.data_ptr(), batch, rows // batch, nh, nkv, hd, max_len,
                                   float(scale if scale is not None else hd ** -0.5), ws.data_ptr(), ws.numel(),
                                   _stream(q.device))
    _lib.check(st, "eptq decode_attention")
    return out


_lm_ws: Dict[tuple, torch.Tensor] = {}


def lm_head_argmax(x: torch.Tensor, weight: torch.Tensor, norm_weight: Optional[torch.Tensor] = None,
                   eps: float = 0.0, want_logits: bool = False, tokens: Optional[torch.Tensor] = None):
    """Greedy pick through the un-quantized output projection (eptq_lm_head_argmax): x (B, H) fp16, weight
    (V, H) fp16 -> int64 tokens (B,), the first index of the maximum of fp16(weight @ x_b).  `norm_weight`
    applies the model's final RMSNorm to x on the way in.  Returns (tokens, logits or None)."""
    _need(x=x, weight=weight, norm_weight=norm_weight, tokens=tokens)
    if x.dtype != torch.float16 or weight.dtype != torch.float16:
        raise RuntimeError("eptq_b200: lm_head_argmax takes fp16 tensors")
    lib = _lib.load()
    B, H = x.shape
    V = weight.shape[0]
    need = lib.eptq_lm_head_workspace_bytes(B)
    if need == 0:
        raise RuntimeError("eptq_b200: lm_head_argmax takes 1..4 rows")
    key = (x.device, torch.cuda.current_stream(x.device).cuda_stream)
    ws = _lm_ws.get(key)
    if ws is None or ws.numel() < need:
        ws = _lm_ws[key] = torch.zeros(need, dtype=torch.uint8, device=x.device)
    tokens = torch.empty(B, dtype=torch.int64, device=x.device) if tokens is None else tokens
    logits = torch.empty((B, V), dtype=torch.float16, device=x.device) if want_logits else None
    st = lib.eptq_lm_head_argmax(weight.data_ptr(), x.data_ptr(), None if norm_weight is None else norm_weight.data_ptr(),
                                 float(eps), None if logits is None else logits.data_ptr(), tokens.data_ptr(),
                                 V, H, B, ws.data_ptr(), ws.numel(), _stream(x.device))
    _lib.check(st, "eptq lm_head_argmax")
    return tokens, logits
