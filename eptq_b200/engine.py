"""Decode engine for LLaMA-architecture models whose decoder linears are EPTQLinear modules.

The reference decodes through the HuggingFace forward wrapped in torch.compile and CUDA graphs
(bench_decode.py:35-83, 149).  Here the per-token step is written out once with static shapes and
captured into ONE CUDA graph that also advances the position and feeds the picked token back, so a
decoded token costs one graph launch and no host work.  Three statements of the same step:

* batch 1, one GPU, E8-D4: per decoder layer the attention kernel and four launches of the streaming GEMV --
  o (+ residual), gate/up (RMSNorm folded in), down (SiLU(gate)*up formed as it reads its input, + residual),
  the next layer's q/k/v (RMSNorm folded in, rotary embedding and cache append in the epilogue); with
  `one_launch_per_layer` the four become the phases of ONE chained launch -- then the final norm, lm_head and
  greedy pick in the library's own kernel;
* batch <= 2 otherwise (E8, tensor parallel): the same work as separate grouped launches;
* anything else, and the prefill: RMSNorm, grouped q/k/v, rotary embedding + cache append, attention, o,
  RMSNorm, grouped gate/up, SiLU*up, down as separate kernels (many tokens: the linears then take the
  tensor-core GEMM path).

Tensor parallelism: with a process group, q/k/v/gate/up hold this rank's output rows (its attention
heads) and o/down this rank's input columns.  Their partial outputs are summed by the push all-reduce
kernel (peer stores, replayed inside the token's graph) when a `PushAllReduce` is given, by NCCL
otherwise and for prefill-sized tensors.  Embedding, norms and lm_head are replicated.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Callable, Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn.functional as F

from .kernels.linear import EPTQLinear, forward_group


@dataclass
class DecoderLayerWeights:
    """The seven linears (any callables mapping (T, in) -> (T, out)) and two norm weights of one layer."""
    q: Callable
    k: Callable
    v: Callable
    o: Callable
    gate: Callable
    up: Callable
    down: Callable
    input_norm: torch.Tensor
    post_norm: torch.Tensor


def apply_group(layers: Sequence[Callable], x: torch.Tensor) -> List[torch.Tensor]:
    """layers[i](x) for all i; one kernel launch when the layers are EPTQLinear modules of one codebook
    and the batch is small enough for the persistent GEMV, otherwise one call per layer."""
    if (x.is_cuda and x.shape[0] <= 16 and all(isinstance(l, EPTQLinear) for l in layers)
            and all(l.quantizer_type == layers[0].quantizer_type and l.S_group is None
                    and l.in_features % 32 == 0 for l in layers)):
        try:
            return forward_group(list(layers), [x] * len(layers))
        except RuntimeError:
            pass                                   # not eligible as one launch (e.g. a warped E8 table)
    return [l(x) for l in layers]


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    d = x.shape[-1] // 2
    return torch.cat((-x[..., d:], x[..., :d]), dim=-1)


class LlamaDecodeEngine:
    """Static-shape forward of a LLaMA-style decoder stack with a preallocated key/value cache."""

    def __init__(self, layers: List[DecoderLayerWeights], embed: torch.Tensor, final_norm: torch.Tensor,
                 lm_head: torch.Tensor, inv_freq: torch.Tensor, rms_eps: float, head_dim: int,
                 n_heads: int, n_kv_heads: int, max_len: int, batch: int = 1,
                 rope_scaling: float = 1.0, tp_group=None, comm=None):
        self.layers = layers
        self.comm = comm                 # eptq_b200.comm.PushAllReduce, or None for NCCL
        self.embed, self.final_norm, self.lm_head = embed, final_norm, lm_head
        self.inv_freq = inv_freq.float()
        self.eps, self.head_dim = float(rms_eps), int(head_dim)
        self.n_heads, self.n_kv_heads = int(n_heads), int(n_kv_heads)      # per rank
        self.max_len, self.batch = int(max_len), int(batch)
        self.rope_scaling = float(rope_scaling)
        self.tp_group = tp_group
        dev, dt = embed.device, embed.dtype
        self.device, self.dtype = dev, dt
        shape = (len(layers), self.batch, self.n_kv_heads, self.max_len, self.head_dim)
        self.k_cache = torch.zeros(shape, dtype=dt, device=dev)
        self.v_cache = torch.zeros(shape, dtype=dt, device=dev)
        self.key_index = torch.arange(self.max_len, device=dev)
        # state of the captured step
        self.token = torch.zeros((self.batch, 1), dtype=torch.long, device=dev)
        self.position = torch.zeros((1,), dtype=torch.long, device=dev)
        self.next_token = torch.zeros((self.batch,), dtype=torch.long, device=dev)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self._pick: Optional[torch.Tensor] = None     # where a fused step writes its token (set inside _step)
        self._fused = None           # descriptors for the fully fused one-token step, False if not eligible
        # Batch-1 decode with the streaming kernel: the four dependent stages of a layer (o, gate/up, down, next
        # q/k/v) as four stream-ordered launches of the same kernel (default), or as ONE chained launch.  Measured
        # on B200, Llama-2-7B shapes: 507 against 470 tokens/s -- a kernel boundary under programmatic dependent
        # launch costs less than a phase boundary inside the launch (ticket, finalize, counter, poll).
        self.one_launch_per_layer = False

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_model(cls, model, max_len: int, batch: int = 1, tp_group=None) -> "LlamaDecodeEngine":
        """Engine over the modules of a LLaMA-style HuggingFace model (as returned by
        load_quantized_model); weights are shared, not copied."""
        core = model.model
        cfg = model.config
        head_dim = getattr(cfg, "head_dim", None) or cfg.hidden_size // cfg.num_attention_heads
        layers = []
        for layer in core.layers:
            a, m = layer.self_attn, layer.mlp
            layers.append(DecoderLayerWeights(a.q_proj, a.k_proj, a.v_proj, a.o_proj, m.gate_proj, m.up_proj,
                                              m.down_proj, layer.input_layernorm.weight.data,
                                              layer.post_attention_layernorm.weight.data))
        q0, k0 = core.layers[0].self_attn.q_proj, core.layers[0].self_attn.k_proj
        rot = core.rotary_emb
        return cls(layers, core.embed_tokens.weight.data, core.norm.weight.data, model.lm_head.weight.data,
                   rot.inv_freq.to(core.embed_tokens.weight.device), cfg.rms_norm_eps, head_dim,
                   q0.out_features // head_dim, k0.out_features // head_dim, max_len, batch,
                   rope_scaling=float(getattr(rot, "attention_scaling", 1.0)), tp_group=tp_group)

    # ---- the step -----------------------------------------------------------------------------
    def _norm(self, x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return F.rms_norm(x, (x.shape[-1],), w, self.eps)

    def _reduce(self, y: torch.Tensor) -> torch.Tensor:
        """Sum the partial outputs of a row-parallel layer over the tensor-parallel group: the one-shot
        push kernel for decode-sized vectors when `self.comm` is set, NCCL otherwise (prefill)."""
        if self.tp_group is not None:
            if self.comm is not None and y.numel() <= self.comm.n_max and y.numel() % 8 == 0:
                self.comm.all_reduce_(y)
            else:
                torch.distributed.all_reduce(y, group=self.tp_group)
        return y

    def forward(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """ids (B, T) token ids, positions (T,) their cache positions (int64 device tensor).  Writes keys
        and values at `positions`, attends to every cached position <= its own, returns logits (B, T, V).
        CUDA fp16 only: the elementwise work runs in this package's fused kernels."""
        if not ids.is_cuda or self.dtype != torch.float16:
            raise RuntimeError("LlamaDecodeEngine.forward runs on CUDA fp16 weights only "
                               "(forward_reference is the plain PyTorch statement of the same step)")
        from .kernels import glue
        B, T = ids.shape
        hd, nh, nkv = self.head_dim, self.n_heads, self.n_kv_heads
        if T == 1 and B <= 2 and hd == 128 and (self.tp_group is None or self.comm is not None) and self._fusable():
            if B == 1 and self.tp_group is None and self._chainable():
                return self._forward_chained_decode(ids, positions)
            return self._forward_fused_decode(ids, positions)
        x = F.embedding(ids, self.embed).reshape(B * T, -1)                        # fresh tensor, updated in place
        fused_attention = T <= 8 and hd in (64, 128)
        mask = None if fused_attention else (self.key_index[None, :] <= positions[:, None])[None, None]
        delta = None
        for li, L in enumerate(self.layers):
            hn = glue.add_rmsnorm(x, L.input_norm, self.eps, delta)                 # x += previous MLP output
            q, k, v = apply_group((L.q, L.k, L.v), hn)
            kc, vc = self.k_cache[li], self.v_cache[li]
            glue.rope_append(q, k, v, kc, vc, positions, self.inv_freq, B, self.rope_scaling)
            if fused_attention:
                att = glue.decode_attention(q, kc, vc, positions, B)
            else:
                qh = q.reshape(B, T, nh, hd).transpose(1, 2)
                if nkv != nh:
                    kc = kc.repeat_interleave(nh // nkv, dim=1)
                    vc = vc.repeat_interleave(nh // nkv, dim=1)
                att = F.scaled_dot_product_attention(qh, kc, vc, attn_mask=mask)
                att = att.transpose(1, 2).reshape(B * T, nh * hd)
            hn = glue.add_rmsnorm(x, L.post_norm, self.eps, self._reduce(L.o(att)))
            gate, up = apply_group((L.gate, L.up), hn)
            delta = self._reduce(L.down(glue.silu_mul(gate, up)))
        hn = glue.add_rmsnorm(x, self.final_norm, self.eps, delta)
        return F.linear(hn, self.lm_head).reshape(B, T, -1)

    # ---- one token, everything fused into the GEMV launches -----------------------------------------
    def _fusable(self) -> bool:
        if self._fused is None:
            mods = [m for L in self.layers for m in (L.q, L.k, L.v, L.o, L.gate, L.up, L.down)]
            ok = all(isinstance(m, EPTQLinear) and m.quantizer_type == mods[0].quantizer_type and m.S_group is None
                     and m.in_features % 32 == 0 and m.out_features % 128 == 0 for m in mods)
            ok = ok and all(m._codebook is mods[0]._codebook for m in mods)      # one table per launch
            if ok and mods[0].quantizer_type == "e8_lattice":
                ok = bool(mods[0].descriptor().table_packed)        # E8 needs a table that packs
            self._fused = self._build_fused() if ok else False
        return self._fused is not False

    def _build_fused(self):
        """Per layer: descriptors of q/k/v and gate/up whose column scales carry the norm weight
        (h' = h * w, so that the kernel only needs the row factor of the RMSNorm), plus o and down."""
        from .kernels import h_absmax
        plan = []
        for L in self.layers:
            keep = []

            def folded(mods, w):
                out = []
                for m in mods:
                    h2 = (m.h.float() * w.float()).to(torch.float16).contiguous()
                    d = m.descriptor()
                    d.h = h2.data_ptr()
                    d.h_absmax = h_absmax(h2)
                    keep.append(h2)
                    out.append(d)
                return out
            plan.append({"qkv": folded((L.q, L.k, L.v), L.input_norm), "o": [L.o.descriptor()],
                         "gate_up": folded((L.gate, L.up), L.post_norm), "down": [L.down.descriptor()],
                         "keep": keep})
        return plan

    def _forward_fused_decode(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """Six launches per decoder layer: q/k/v (RMSNorm folded in; rotary embedding and the cache
        append done by the finalizing warps), attention, o (+ residual), gate/up (RMSNorm folded in),
        SiLU*up, down (+ residual).  Tensor-parallel: o and down store partial sums and the push
        all-reduce adds them to the residual stream (eight launches).  (gate/up -> down as two phases of one
        chained launch was measured here too: 425 against 433 tokens/s at two GPUs, so the separate launches stay.)"""
        from . import _lib
        from .kernels import glue, linear_forward_chain, linear_forward_group
        B = ids.shape[0]
        hd, nh, nkv = self.head_dim, self.n_heads, self.n_kv_heads
        x = F.embedding(ids, self.embed).reshape(B, -1).contiguous()                # residual stream, updated in place
        pos_ptr, freq_ptr = positions.data_ptr(), self.inv_freq.data_ptr()

        def fus(x_op=_lib.X_PLAIN, y_op=_lib.Y_STORE, residual=None, x_aux=None):
            f = _lib.EptqFusion()
            f.x_op, f.y_op, f.norm_eps, f.rope_scaling, f.max_len = x_op, y_op, self.eps, self.rope_scaling, self.max_len
            f.residual = None if residual is None else residual.data_ptr()
            f.x_aux = None if x_aux is None else x_aux.data_ptr()
            f.position, f.inv_freq = pos_ptr, freq_ptr
            return f
        qkv_f = [fus(_lib.X_RMSNORM, _lib.Y_ROPE), fus(_lib.X_RMSNORM, _lib.Y_ROPE_TO_CACHE),
                 fus(_lib.X_RMSNORM, _lib.Y_TO_CACHE)]
        gu_f = [fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM)]
        res_f = [fus(y_op=_lib.Y_ADD_RESIDUAL, residual=x)]
        for li, (L, P) in enumerate(zip(self.layers, self._fused)):
            kc, vc = self.k_cache[li], self.v_cache[li]
            q = linear_forward_group(P["qkv"], [x, x, x], [nh * hd, 0, 0], fusions=qkv_f, ys=[None, kc, vc])[0]
            att = glue.decode_attention(q, kc, vc, positions, B)
            if self.tp_group is None:
                linear_forward_group(P["o"], [att], [0], fusions=res_f, ys=[x])
            else:                                   # partial sums: the reduction adds them to the residual stream
                self.comm.all_reduce_(linear_forward_group(P["o"], [att], [L.o.out_features])[0], residual=x)
            gate, up = linear_forward_group(P["gate_up"], [x, x], [L.gate.out_features, L.up.out_features], fusions=gu_f)
            d = P["down"][0]
            if B == 1 and bool(d.table8) and d.table8_scale > 0 and d.N % 64 == 0 and d.N <= 25600:
                # the streaming kernel forms silu(gate) * up as it reads its input: no launch for it
                f = fus(_lib.X_SILU_MUL, x_aux=up) if self.tp_group is not None else \
                    fus(_lib.X_SILU_MUL, _lib.Y_ADD_RESIDUAL, residual=x, x_aux=up)
                out = linear_forward_chain(P["down"], [0], [gate], [0 if self.tp_group is None else L.down.out_features],
                                           [f], ys=[x] if self.tp_group is None else None)
                if self.tp_group is not None:
                    self.comm.all_reduce_(out[0], residual=x)
                continue
            act = glue.silu_mul(gate, up)
            if self.tp_group is None:
                linear_forward_group(P["down"], [act], [0], fusions=res_f, ys=[x])
            else:
                self.comm.all_reduce_(linear_forward_group(P["down"], [act], [L.down.out_features])[0], residual=x)
        return self._head(x, B)

    # ---- one token, two launches per decoder layer ----------------------------------------------
    def _chainable(self) -> bool:
        """Batch-1 decode on one GPU with layers the streaming kernel takes (E8-D4 on the lattice, in_features a
        multiple of 64): attention, then ONE chained launch for o -> gate/up -> down -> the next layer's q/k/v."""
        if getattr(self, "_chain_ok", None) is None:
            ok = self._fusable()
            if ok:
                for P in self._fused:
                    for d in P["qkv"] + P["o"] + P["gate_up"] + P["down"]:
                        ok = ok and bool(d.table8) and d.table8_scale > 0 and d.N % 64 == 0 and d.N <= 25600
            self._chain_ok = bool(ok)
        return self._chain_ok

    def _forward_chained_decode(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """q/k/v of the first layer, then per layer: attention and one chained launch -- o (+ residual), gate/up
        (RMSNorm folded in), down on silu(gate)*up (+ residual), q/k/v of the next layer (RMSNorm folded in,
        rotary embedding, cache append)."""
        from . import _lib
        from .kernels import glue, linear_forward_chain, linear_forward_group
        hd, nh = self.head_dim, self.n_heads
        x = F.embedding(ids, self.embed).reshape(1, -1).contiguous()                # residual stream, updated in place
        pos_ptr, freq_ptr = positions.data_ptr(), self.inv_freq.data_ptr()
        inter = self.layers[0].gate.out_features
        gate = torch.empty((1, inter), dtype=torch.float16, device=x.device)
        up = torch.empty_like(gate)
        qs = [torch.empty((1, nh * hd), dtype=torch.float16, device=x.device) for _ in range(2)]

        def fus(x_op=_lib.X_PLAIN, y_op=_lib.Y_STORE, residual=None, x_aux=None):
            f = _lib.EptqFusion()
            f.x_op, f.y_op, f.norm_eps, f.rope_scaling, f.max_len = x_op, y_op, self.eps, self.rope_scaling, self.max_len
            f.residual = None if residual is None else residual.data_ptr()
            f.x_aux = None if x_aux is None else x_aux.data_ptr()
            f.position, f.inv_freq = pos_ptr, freq_ptr
            return f
        qkv_f = [fus(_lib.X_RMSNORM, _lib.Y_ROPE), fus(_lib.X_RMSNORM, _lib.Y_ROPE_TO_CACHE),
                 fus(_lib.X_RMSNORM, _lib.Y_TO_CACHE)]
        mlp_f = [fus(y_op=_lib.Y_ADD_RESIDUAL, residual=x), fus(_lib.X_RMSNORM), fus(_lib.X_RMSNORM),
                 fus(_lib.X_SILU_MUL, _lib.Y_ADD_RESIDUAL, residual=x, x_aux=up)]
        n_layers = len(self.layers)
        linear_forward_group(self._fused[0]["qkv"], [x, x, x], [0, 0, 0], fusions=qkv_f,
                             ys=[qs[0], self.k_cache[0], self.v_cache[0]])
        for li, P in enumerate(self._fused):
            q = qs[li & 1]
            att = glue.decode_attention(q, self.k_cache[li], self.v_cache[li], positions, 1)
            descs = P["o"] + P["gate_up"] + P["down"]
            phases = [0, 1, 1, 2]
            xs = [att, x, x, gate]
            ys = [x, gate, up, x]
            fz = list(mlp_f)
            if li + 1 < n_layers:
                descs = descs + self._fused[li + 1]["qkv"]
                phases += [3, 3, 3]
                xs += [x, x, x]
                ys += [qs[(li + 1) & 1], self.k_cache[li + 1], self.v_cache[li + 1]]
                fz += qkv_f
            if self.one_launch_per_layer:
                linear_forward_chain(descs, phases, xs, [0] * len(descs), fz, ys=ys)
            else:                                            # the same stages as stream-ordered launches
                lo = 0
                for hi in range(1, len(descs) + 1):
                    if hi == len(descs) or phases[hi] != phases[lo]:
                        linear_forward_chain(descs[lo:hi], [0] * (hi - lo), xs[lo:hi], [0] * (hi - lo), fz[lo:hi], ys=ys[lo:hi])
                        lo = hi
        return self._head(x, 1)

    def _head(self, x: torch.Tensor, B: int) -> torch.Tensor:
        """Final RMSNorm and lm_head of a one-token step.  While a step is being taken (`_pick` set by `_step`),
        the library's fused norm + projection + greedy pick writes the next token and the logits are not
        materialised; otherwise logits (B, 1, V)."""
        from .kernels import glue
        H = x.shape[-1]
        if self._pick is not None and B <= 4 and H % 256 == 0 and H <= 8192:
            glue.lm_head_argmax(x, self.lm_head, self.final_norm, self.eps, tokens=self._pick)
            return None
        hn = glue.add_rmsnorm(x, self.final_norm, self.eps)
        return F.linear(hn, self.lm_head).reshape(B, 1, -1)

    def forward_reference(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        """The same step in plain PyTorch ops, on any device and dtype: what `forward` is tested against,
        and itself tested against the HuggingFace forward."""
        B, T = ids.shape
        hd, nh, nkv = self.head_dim, self.n_heads, self.n_kv_heads
        x = F.embedding(ids, self.embed).reshape(B * T, -1)
        ang = positions.float()[:, None] * self.inv_freq[None, :]                   # (T, hd/2)
        ang = torch.cat((ang, ang), dim=-1)
        cos = (ang.cos() * self.rope_scaling).to(self.dtype)[None, None]            # (1, 1, T, hd)
        sin = (ang.sin() * self.rope_scaling).to(self.dtype)[None, None]
        mask = (self.key_index[None, :] <= positions[:, None])[None, None]          # (1, 1, T, max_len)
        for li, L in enumerate(self.layers):
            hn = self._norm(x, L.input_norm)
            q, k, v = (f(hn) for f in (L.q, L.k, L.v))
            q = q.reshape(B, T, nh, hd).transpose(1, 2)
            k = k.reshape(B, T, nkv, hd).transpose(1, 2)
            v = v.reshape(B, T, nkv, hd).transpose(1, 2)
            q = q * cos + rotate_half(q) * sin
            k = k * cos + rotate_half(k) * sin
            kc, vc = self.k_cache[li], self.v_cache[li]
            kc.index_copy_(2, positions, k)
            vc.index_copy_(2, positions, v)
            if nkv != nh:
                kc = kc.repeat_interleave(nh // nkv, dim=1)
                vc = vc.repeat_interleave(nh // nkv, dim=1)
            att = F.scaled_dot_product_attention(q, kc, vc, attn_mask=mask)
            att = att.transpose(1, 2).reshape(B * T, nh * hd)
            x = x + self._reduce(L.o(att))
            hn = self._norm(x, L.post_norm)
            x = x + self._reduce(L.down(F.silu(L.gate(hn)) * L.up(hn)))
        x = self._norm(x, self.final_norm)
        return F.linear(x, self.lm_head).reshape(B, T, -1)

    # ---- driving it ---------------------------------------------------------------------------
    @torch.no_grad()
    def prefill(self, ids: torch.Tensor) -> torch.Tensor:
        """Run the prompt (B, T) through the stack, fill the cache, set up the decode state; returns the
        first generated token (greedy)."""
        B, T = ids.shape
        if B != self.batch or T >= self.max_len:
            raise ValueError("prompt does not fit the engine's batch / cache length")
        pos = torch.arange(T, device=self.device)
        logits = self._fwd(ids, pos)
        self._check_device_status("prefill")
        first = logits[:, -1].argmax(dim=-1)
        self.token.copy_(first[:, None])
        self.position.fill_(T)
        return first

    def _check_device_status(self, what: str) -> None:
        """A kernel whose bounded device-side wait ran out (prefill GEMM, streaming or chained GEMV) leaves a code
        in the status word of the scratch it used: read it (one stream synchronisation) and raise."""
        if self.device.type != "cuda":
            return
        from . import _lib
        from .kernels import workspace_status_all
        code = workspace_status_all(self.device)
        if code != 0:
            _lib.check(code, f"eptq_b200 {what} (device-side wait)")

    def _fwd(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        fused = ids.is_cuda and self.dtype == torch.float16
        return self.forward(ids, positions) if fused else self.forward_reference(ids, positions)

    def _step(self) -> None:
        self._pick = self.next_token if (self.token.is_cuda and self.dtype == torch.float16) else None
        try:
            logits = self._fwd(self.token, self.position)
        finally:
            self._pick = None
        if logits is None:                                   # the fused head already wrote next_token
            self.token.copy_(self.next_token[:, None])
            self.position.add_(1)
            return
        nxt = logits[:, -1].argmax(dim=-1)
        self.next_token.copy_(nxt)
        self.token.copy_(nxt[:, None])
        self.position.add_(1)

    @torch.no_grad()
    def capture(self) -> None:
        """Capture one decode step into a CUDA graph.  The cache contents and the decode state are
        restored afterwards, so this may be called between prefill and decode."""
        saved = (self.token.clone(), self.position.clone())
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):                                   # allocate scratch, start NCCL, warm caches
                self._step()
                self.token.copy_(saved[0]); self.position.copy_(saved[1])
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=side):       # same stream: the scratch made in the warm-up is reused
            self._step()
        self.graph = graph
        self.token.copy_(saved[0]); self.position.copy_(saved[1])
        torch.cuda.synchronize(self.device)

    @torch.no_grad()
    def decode(self, ids: torch.Tensor, max_new_tokens: int, use_graph: bool = True
               ) -> Tuple[torch.Tensor, Dict[str, float]]:
        """Greedy decode.  Returns (tokens (B, max_new_tokens), timings) with the reference's protocol
        (bench_decode.py:56-71): prefill excluded, tokens/s = (new tokens - 1) * batch / loop time."""
        if ids.shape[1] + max_new_tokens > self.max_len:
            raise ValueError("prompt + new tokens exceed the cache length")
        if use_graph and self.graph is None:
            self.prefill(ids)                                    # realistic state for the warm-up steps
            self.capture()
        torch.cuda.synchronize(self.device)
        t0 = time.perf_counter()
        first = self.prefill(ids)
        torch.cuda.synchronize(self.device)
        t1 = time.perf_counter()
        out = torch.empty((self.batch, max_new_tokens), dtype=torch.long, device=self.device)
        out[:, 0] = first
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for i in range(1, max_new_tokens):
            if use_graph:
                self.graph.replay()
            else:
                self._step()
            out[:, i] = self.next_token
        stop.record()
        torch.cuda.synchronize(self.device)
        dev_s = start.elapsed_time(stop) * 1e-3
        n = max(max_new_tokens - 1, 1) * self.batch
        self._check_device_status("decode")
        return out, {"prefill_s": t1 - t0, "decode_s": dev_s, "tokens_per_s": n / max(dev_s, 1e-9),
                     "ms_per_token": 1e3 * dev_s / max(max_new_tokens - 1, 1)}


@dataclass
class OPTLayerWeights:
    """The six linears (with their biases inside) and the two LayerNorms of one OPT decoder layer."""
    q: Callable
    k: Callable
    v: Callable
    o: Callable
    fc1: Callable
    fc2: Callable
    ln1_w: torch.Tensor
    ln1_b: torch.Tensor
    ln2_w: torch.Tensor
    ln2_b: torch.Tensor


class OPTDecodeEngine(LlamaDecodeEngine):
    """The same engine for OPT-style decoders (models/opt.py:14-16, 62-68 of the reference; pre-LayerNorm
    variants, i.e. every published size except 350m): learned positions, LayerNorm with bias, ReLU MLP, biases
    in every projection, no rotary embedding.  One token = one CUDA graph as in the LLaMA engine (prefill,
    capture, decode and the greedy state are inherited).  The quantized projections run in this package's
    kernels (q/k/v as one grouped launch, single-query attention over the cache); LayerNorm, ReLU and the
    residual adds are PyTorch elementwise ops inside the captured step."""

    def __init__(self, layers: List[OPTLayerWeights], embed: torch.Tensor, pos_embed: torch.Tensor,
                 final_ln_w: torch.Tensor, final_ln_b: torch.Tensor, lm_head: torch.Tensor, head_dim: int,
                 n_heads: int, max_len: int, batch: int = 1, ln_eps: float = 1e-5, pos_offset: int = 2):
        super().__init__(layers, embed, final_ln_w, lm_head, torch.zeros(head_dim // 2), ln_eps, head_dim,
                         n_heads, n_heads, max_len, batch)
        self.pos_embed, self.pos_offset = pos_embed, int(pos_offset)
        self.final_ln_b = final_ln_b
        self._fused = False                                   # the fused LLaMA steps do not apply

    @classmethod
    def from_model(cls, model, max_len: int, batch: int = 1, tp_group=None) -> "OPTDecodeEngine":
        """Engine over the modules of a HuggingFace OPT model (as returned by load_quantized_model); weights are
        shared, not copied."""
        if tp_group is not None:
            raise NotImplementedError("the OPT engine is single-GPU")
        dec = model.model.decoder
        cfg = model.config
        if not cfg.do_layer_norm_before or dec.project_in is not None or dec.project_out is not None:
            raise NotImplementedError("post-LayerNorm / projected-embedding OPT variants (opt-350m) are not covered")
        layers = []
        for layer in dec.layers:
            a = layer.self_attn
            layers.append(OPTLayerWeights(a.q_proj, a.k_proj, a.v_proj, a.out_proj, layer.fc1, layer.fc2,
                                          layer.self_attn_layer_norm.weight.data, layer.self_attn_layer_norm.bias.data,
                                          layer.final_layer_norm.weight.data, layer.final_layer_norm.bias.data))
        head_dim = cfg.hidden_size // cfg.num_attention_heads
        return cls(layers, dec.embed_tokens.weight.data, dec.embed_positions.weight.data,
                   dec.final_layer_norm.weight.data, dec.final_layer_norm.bias.data, model.lm_head.weight.data,
                   head_dim, cfg.num_attention_heads, max_len, batch,
                   ln_eps=float(dec.final_layer_norm.eps), pos_offset=int(getattr(dec.embed_positions, "offset", 2)))

    def _ln(self, x: torch.Tensor, w: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
        return F.layer_norm(x, (x.shape[-1],), w, b, self.eps)

    def _stack(self, ids: torch.Tensor, positions: torch.Tensor, kernels: bool) -> torch.Tensor:
        B, T = ids.shape
        hd, nh = self.head_dim, self.n_heads
        x = (F.embedding(ids, self.embed) + F.embedding(positions + self.pos_offset, self.pos_embed)[None]).reshape(B * T, -1)
        fused_attention = kernels and T <= 8 and hd in (64, 128)
        mask = None if fused_attention else (self.key_index[None, :] <= positions[:, None])[None, None]
        if kernels:
            from .kernels import glue
        for li, L in enumerate(self.layers):
            hn = self._ln(x, L.ln1_w, L.ln1_b)
            q, k, v = apply_group((L.q, L.k, L.v), hn) if kernels else [f(hn) for f in (L.q, L.k, L.v)]
            kc, vc = self.k_cache[li], self.v_cache[li]
            kc.index_copy_(2, positions, k.reshape(B, T, nh, hd).transpose(1, 2))
            vc.index_copy_(2, positions, v.reshape(B, T, nh, hd).transpose(1, 2))
            if fused_attention:
                att = glue.decode_attention(q.contiguous(), kc, vc, positions, B)
            else:
                att = F.scaled_dot_product_attention(q.reshape(B, T, nh, hd).transpose(1, 2), kc, vc, attn_mask=mask)
                att = att.transpose(1, 2).reshape(B * T, nh * hd)
            x = x + L.o(att)
            hn = self._ln(x, L.ln2_w, L.ln2_b)
            x = x + L.fc2(F.relu(L.fc1(hn)))
        x = self._ln(x, self.final_norm, self.final_ln_b)
        return F.linear(x, self.lm_head).reshape(B, T, -1)

    def forward(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        if not ids.is_cuda or self.dtype != torch.float16:
            raise RuntimeError("OPTDecodeEngine.forward runs on CUDA fp16 weights only "
                               "(forward_reference is the plain PyTorch statement of the same step)")
        return self._stack(ids, positions, kernels=True)

    def forward_reference(self, ids: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
        return self._stack(ids, positions, kernels=False)


def decode_engine_for(model, max_len: int, batch: int = 1, tp_group=None) -> LlamaDecodeEngine:
    """The engine class that matches a HuggingFace model's architecture (OPT or LLaMA-style)."""
    kind = str(getattr(model.config, "model_type", "")).lower()
    cls = OPTDecodeEngine if kind == "opt" else LlamaDecodeEngine
    return cls.from_model(model, max_len, batch, tp_group=tp_group)


def synthetic_llama_engine(hidden: int, intermediate: int, n_layers: int, n_heads: int, n_kv_heads: int,
                           vocab: int, quantizer_type: str, codebook: torch.Tensor, max_len: int, batch: int = 1,
                           device: str = "cuda", seed: int = 42, outlier_frac: float = 0.002,
                           tp_rank: int = 0, tp_size: int = 1, tp_group=None, init_std: float = 0.02,
                           rope_theta: float = 10000.0, rms_eps: float = 1e-5, comm=None) -> LlamaDecodeEngine:
    """Random-init model of a LLaMA architecture, every decoder linear a synthetic quantized layer
    (make_layer), sharded for this rank when tp_size > 1.  Real checkpoints need the model hub; the
    shapes and value distributions are what matters for throughput.  Row scales carry an extra factor
    so that activations stay finite in fp16 through the whole stack; norms are ones, embeddings and
    lm_head N(0, init_std)."""
    from .parallel import shard_layer
    from .synthetic import make_layer

    head_dim = hidden // n_heads
    shapes = {"q_proj": (n_heads * head_dim, hidden), "k_proj": (n_kv_heads * head_dim, hidden),
              "v_proj": (n_kv_heads * head_dim, hidden), "o_proj": (hidden, n_heads * head_dim),
              "gate_proj": (intermediate, hidden), "up_proj": (intermediate, hidden),
              "down_proj": (hidden, intermediate)}
    dev = torch.device(device)
    codebook = codebook.to(dev)
    layers = []
    for lid in range(n_layers):
        mods = {}
        for k, (name, (o, i)) in enumerate(shapes.items()):
            qd = make_layer(o, i, seed=seed + 1000 * lid + k, outlier_frac=outlier_frac, device=str(dev),
                            scale_sigma=0.05)
            # wider and deeper stacks get proportionally smaller row scales, so that the residual stream of a
            # random-init model stays finite in fp16 (no effect at hidden size 4096 and 32 layers or fewer)
            damp = (4096.0 / max(hidden, 4096)) ** 0.5 * (32.0 / max(n_layers, 32)) ** 0.5
            qd.g = (qd.g.float() * (init_std * 1.5 * damp)).to(torch.float16)
            qd = shard_layer(qd, name, tp_rank, tp_size)
            mods[name] = EPTQLinear.from_quantized_data(qd, codebook, quantizer_type)
        ones = torch.ones(hidden, dtype=torch.float16, device=dev)
        layers.append(DecoderLayerWeights(mods["q_proj"], mods["k_proj"], mods["v_proj"], mods["o_proj"],
                                          mods["gate_proj"], mods["up_proj"], mods["down_proj"], ones, ones.clone()))
    gen = torch.Generator(device=dev).manual_seed(seed)
    embed = (torch.randn((vocab, hidden), generator=gen, device=dev) * init_std).to(torch.float16)
    head = (torch.randn((vocab, hidden), generator=gen, device=dev) * init_std).to(torch.float16)
    inv_freq = 1.0 / (rope_theta ** (torch.arange(0, head_dim, 2, device=dev).float() / head_dim))
    return LlamaDecodeEngine(layers, embed, torch.ones(hidden, dtype=torch.float16, device=dev), head, inv_freq,
                             rms_eps, head_dim, n_heads // tp_size, n_kv_heads // tp_size, max_len, batch,
                             tp_group=tp_group, comm=comm)


ARCHITECTURES = {      # name -> hidden, intermediate, layers, heads, kv heads, vocabulary
    "llama2-7b": (4096, 11008, 32, 32, 32, 32000),
    "llama3-8b": (4096, 14336, 32, 32, 8, 128256),
    "llama2-70b": (8192, 28672, 80, 64, 8, 32000),
    "tiny": (256, 704, 2, 8, 8, 1024),
}


def _main():
    """Whole-model greedy decode of a random-init architecture; under torchrun, tensor-parallel over
    all ranks.  Prints one JSON line (rank 0)."""
    import argparse
    import json
    import os

    from .quantizers import E8D4Quantizer, E8LatticeQuantizer

    ap = argparse.ArgumentParser()
    ap.add_argument("--arch", default="llama2-7b", choices=sorted(ARCHITECTURES))
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--quantizer", default="e8_d4", choices=["e8_d4", "e8_lattice"])
    ap.add_argument("--prefill", type=int, default=512)
    ap.add_argument("--new-tokens", type=int, default=128)
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--nccl", action="store_true", help="all-reduce with NCCL instead of the push kernel")
    args = ap.parse_args()

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    group = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
        group = dist.group.WORLD
    hidden, inter, n_layers, heads, kv, vocab = ARCHITECTURES[args.arch]
    n_layers = args.layers or n_layers
    if args.quantizer == "e8_d4":
        table = E8D4Quantizer(radius=1.75).codes
    else:
        q = E8LatticeQuantizer(radius=1.6)
        q.remove_last()
        table = q.points
    comm = None
    if world > 1 and not args.nccl:
        from .comm import PushAllReduce
        try:
            comm = PushAllReduce(group, args.batch * hidden, torch.device("cuda", local))
        except RuntimeError as exc:              # raised on every rank alike: NCCL instead
            if rank == 0:
                print(f"push all-reduce unavailable, using NCCL: {exc}", file=__import__("sys").stderr)
    eng = synthetic_llama_engine(hidden, inter, n_layers, heads, kv, vocab, args.quantizer, table,
                                 max_len=args.prefill + args.new_tokens, batch=args.batch, device=f"cuda:{local}",
                                 tp_rank=rank, tp_size=world, tp_group=group, comm=comm)
    ids = torch.randint(0, vocab, (args.batch, args.prefill), generator=torch.Generator().manual_seed(0)).cuda()
    eng.decode(ids, min(8, args.new_tokens), use_graph=not args.no_graph)          # warm-up (and capture)
    toks, stats = eng.decode(ids, args.new_tokens, use_graph=not args.no_graph)
    if comm is not None:
        comm.check()
    if world > 1:
        stat_t = torch.tensor([stats["decode_s"]], device="cuda")
        torch.distributed.all_reduce(stat_t, op=torch.distributed.ReduceOp.MAX)
        stats["decode_s"] = float(stat_t.item())
        stats["tokens_per_s"] = max(args.new_tokens - 1, 1) * args.batch / stats["decode_s"]
        stats["ms_per_token"] = 1e3 * stats["decode_s"] / max(args.new_tokens - 1, 1)
    if rank == 0:
        print(json.dumps({"arch": args.arch, "layers": n_layers, "quantizer": args.quantizer, "batch": args.batch,
                          "tp": world, "all_reduce": ("none" if world == 1 else "nccl" if comm is None else "push kernel"),
                          "prefill_tokens": args.prefill, "new_tokens": args.new_tokens,
                          "cuda_graph": not args.no_graph, **stats}), flush=True)
    if world > 1:
        torch.cuda.synchronize()
        os._exit(0)


if __name__ == "__main__":
    _main()
