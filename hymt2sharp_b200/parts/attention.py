"""Grouped-query causal attention over the paged cache, as a mixer part.

q, k, v = x·Wq^T, x·Wk^T, x·Wv^T (one fused product); position encoding on q
and k; optional per-head RMSNorm of q and k after it; k, v appended to the
cache; softmax((q·k)/sqrt(d)) over the visible keys; · v; output projection
added to the residual stream
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:38-89).  An optional window limits
the visible keys to the last `window` positions.

Beyond that form, chosen by parameters: values of another width than keys (`value_dim`); a score scale of its own
(`scale`); the q/k norm BEFORE the rotation (`norm_first`), per head with one gain of head_dim entries (`qk_norm` True or
"head") or over a token's whole q (and k) projection with a gain as wide as the projection ("all"); a sink in the softmax
(`sink`: one more term in the denominator, of score 0 and without a value); and a layer without key/value projections of its
own (`own_kv` False), which reads the cache plane of the run that the model's order names for it, with its own queries;
biases of the q, k and v projections (`q_bias`, `k_bias`, `v_bias`: stored vectors, added before the rotation); and a gate
per head (`head_gate`: a stored matrix [heads, hidden]; head h's output is multiplied by sigmoid((W_gate x)_h) in front of
the output projection).
The classic form (none of these) runs the fused and tensor-core kernels; the others run the general kernels, and the
tensor-core attention where it takes the shape.
"""
from __future__ import annotations

import math

import torch

from ..cache.allocator import GroupSpec
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, PartSpec, Prenormed, RotaryEpilogue, build_part, register_part
from .linear import Linear, compute_form

SPLIT_KEYS = 256  # decode: keys per partial, a constant so that the cut depends on nothing else


class GQAAttention:
    graph_safe = True  # its forward only launches kernels on the current stream
    takes_prenormed = True  # x may be a parts.base.Prenormed: the projection applies the norm's row scale itself
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, heads: int, kv_heads: int, head_dim: int, eps: float, qk_norm,
                 position: PartSpec | None, q_proj: str, k_proj: str | None, v_proj: str | None, o_proj: str,
                 q_norm: str | None = None, k_norm: str | None = None, window: int | None = None,
                 value_dim: int | None = None, scale: float | None = None, norm_first: bool = False, sink: bool = False,
                 own_kv: bool = True, q_bias: str | None = None, k_bias: str | None = None, v_bias: str | None = None,
                 head_gate: str | None = None):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if qk_norm not in (False, True, None, "head", "all"):
            raise ValueError(f"qk_norm '{qk_norm}': known are False, 'head' (True) and 'all'")
        self.hidden, self.heads, self.kv_heads, self.head_dim = hidden, heads, kv_heads, head_dim
        self.value_dim = int(value_dim or head_dim)
        self.qk_norm = "head" if qk_norm is True else (qk_norm or None)
        self.eps, self.window = float(eps), int(window or 0)
        self.norm_first, self.sink, self.own_kv = bool(norm_first), bool(sink), bool(own_kv)
        if self.qk_norm == "all" and not self.norm_first:
            raise ValueError("a q/k norm over the whole projection comes before the rotation (norm_first)")
        if self.own_kv and (k_proj is None or v_proj is None):
            raise ValueError("an attention with keys and values of its own needs the names of their projections")
        # the form that the fused projection and the classic kernels know
        biased = q_bias is not None or k_bias is not None or v_bias is not None
        if biased and (q_bias is None or (self.own_kv and (k_bias is None or v_bias is None))):
            raise ValueError("biases come for every projection that the attention has, or for none")
        self.classic = (self.value_dim == head_dim and not self.norm_first and not self.sink and self.own_kv
                        and self.qk_norm != "all" and not biased and head_gate is None)
        if self.classic and (head_dim % 8 or head_dim > 256):   # what the classic kernels take; the tensor-core kernels take 64 and 128
            raise ValueError(f"head_dim {head_dim} must be a multiple of 8, at most 256")
        self.names = dict(q=q_proj, k=k_proj, v=v_proj, o=o_proj, qn=q_norm, kn=k_norm, qb=q_bias, kb=k_bias, vb=v_bias, g=head_gate)
        self.bias = self.gate = None
        self.position = build_part("position", position) if position is not None else None
        self.scale = 1.0 / math.sqrt(head_dim) if scale is None else float(scale)  # src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:64
        self.qkv = self.out = self.out_store = self.q_gain = self.k_gain = None

    # -- what it needs ----------------------------------------------------------
    def tensors(self):
        qd, kd, h, n = self.heads * self.head_dim, self.kv_heads * self.head_dim, self.hidden, self.names
        t = {n["q"]: TensorSpec((qd, h)), n["o"]: TensorSpec((h, self.heads * self.value_dim))}
        if self.own_kv:
            t[n["k"]] = TensorSpec((kd, h))
            t[n["v"]] = TensorSpec((self.kv_heads * self.value_dim, h))
        if self.qk_norm:
            wide = self.qk_norm == "all"
            t[n["qn"]] = TensorSpec((qd if wide else self.head_dim,), init="gain")
            if self.own_kv:
                t[n["kn"]] = TensorSpec((kd if wide else self.head_dim,), init="gain")
        if n["qb"] is not None:
            t[n["qb"]] = TensorSpec((qd,))
            if self.own_kv:
                t[n["kb"]] = TensorSpec((kd,))
                t[n["vb"]] = TensorSpec((self.kv_heads * self.value_dim,))
        if n["g"] is not None:
            t[n["g"]] = TensorSpec((self.heads, h))
        if self.position is not None:
            t.update(self.position.tensors())
        return t

    def cache_need(self):
        kind = "window" if self.window > 0 else "full"
        return GroupSpec(kind, self.kv_heads, self.head_dim, planes=0, window=self.window,
                         value_dim=0 if self.value_dim == self.head_dim else self.value_dim)

    def state_bytes(self) -> int:
        return 0

    def load(self, weights, device, dtype):
        n = self.names
        rows = [weights[n["q"]]] + ([weights[n["k"]], weights[n["v"]]] if self.own_kv else [])
        self.qkv = Linear(compute_form(torch.cat(rows, dim=0), device, dtype), role="qkv" if self.own_kv else "q_proj")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        if n["qb"] is not None:
            self.bias = torch.cat([weights[name].to(device).float().reshape(-1)
                                   for name in ([n["qb"]] + ([n["kb"], n["vb"]] if self.own_kv else []))]).contiguous()
        if n["g"] is not None:
            self.gate = Linear(compute_form(weights[n["g"]], device, dtype), role="head_gate")
        if self.qk_norm:
            self.q_gain = compute_form(weights[n["qn"]], device, dtype)
            self.k_gain = compute_form(weights[n["kn"]], device, dtype) if self.own_kv else None
            if self.k_gain is not None and self.q_gain.dtype != self.k_gain.dtype:
                self.q_gain, self.k_gain = self.q_gain.float(), self.k_gain.float()
        if self.position is not None:
            self.position.load(weights, device, dtype)

    # -- the step ---------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        if not self.classic:
            return self._forward_general(x, residual, ctx, slot, store)
        from ..kernels import fast
        T = ctx.num_tokens
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        # the position encoding in the form that the appending kernels take, or None: it rotates q and k itself
        epilogue = self.position.kernel_epilogue(ctx) if self.position is not None else RotaryEpilogue.none()
        if epilogue is not None and epilogue.rope_dim and epilogue.pairing != "half":
            raise ValueError("the kernels of this attention rotate pairs (i, i + rope_dim/2); its position encoding offers another pairing")
        k_plane, v_plane = ctx.cache.plane(slot.group, slot.plane)
        block_table = ctx.cache.tables[slot.group]
        planes = (k_plane, v_plane) if slot.writes else (None, None)
        q = None
        pre = x if isinstance(x, Prenormed) else None
        if epilogue is not None and x.shape[0] == T:
            # projection, rotation, norm and cache append as one kernel, where the kernels have one for the shape
            q = fast.try_project_rope_kv(pre.normed if pre else x, self.qkv.weight, epilogue, ctx, planes, k_plane.dtype,
                                         block_table, self.q_gain, self.k_gain, self.eps, nh, nkv, d,
                                         row_scale=pre.row_scale() if pre else None)
        if q is None:
            qkv = self.qkv(x, ctx=ctx)
            if epilogue is None:
                self.position.apply(qkv, ctx, nh, nkv, d)
                epilogue = RotaryEpilogue.none()
            q = torch.empty((T, nh * d), dtype=qkv.dtype, device=qkv.device)
            ops.rope_kv(qkv, q, planes[0], planes[1], block_table, ctx.cache.block_tokens, ctx.token_seq, ctx.token_pos,
                        ctx.slot_ids, epilogue.inv_freq, epilogue.rope_dim, self.q_gain, self.k_gain, self.eps, nh, nkv, d)
        out = torch.empty((T, nh * d), dtype=q.dtype, device=q.device)
        self.attend(out, q, k_plane, v_plane, block_table, ctx)
        if ctx.decode and ctx.weights_ahead is not None:
            # the feed-forward's first weights come into L2 beside the output projection and the norm, which leave
            # the memory idle; the request starts once the attention is through (not earlier: its last loads and
            # the folding of its partials are sensitive to traffic)
            ops.prefetch_beside(ctx.weights_ahead)
        if store:
            self.out_store(out, out=residual)
        else:
            self.out.add_then_norm(out, residual, getattr(ctx, "norm_ahead", None), ctx)

    def _forward_general(self, x, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool) -> None:
        """Every form beyond the classic one: the projection as one product, then norm, rotation and cache append in one
        kernel, then the attention, then the output projection."""
        from ..kernels import fast
        if slot.writes != self.own_kv:
            raise ValueError("an attention without key/value projections reads another run's cache plane, and only such a one does")
        T, nh, nkv, d, dv = ctx.num_tokens, self.heads, self.kv_heads, self.head_dim, self.value_dim
        epilogue = self.position.kernel_epilogue(ctx) if self.position is not None else RotaryEpilogue.none()
        if epilogue is None or (epilogue.rope_dim and epilogue.pairing != "half") or epilogue.amplitude != 1.0:
            raise ValueError("the kernels of this attention rotate pairs (i, i + rope_dim/2) by a table of frequencies")
        k_plane, v_plane = ctx.cache.plane(slot.group, slot.plane)
        block_table = ctx.cache.tables[slot.group]
        proj = self.qkv(x, ctx=ctx)
        if self.bias is not None:
            ops.bias_act(proj, self.bias, 0)
        gate = self.gate(x, ctx=ctx) if self.gate is not None else None     # [T, heads], read behind the attention
        q = torch.empty((T, nh * d), dtype=proj.dtype, device=proj.device)
        mode = ops.NORM_NONE if not self.qk_norm else (ops.NORM_ALL_BEFORE if self.qk_norm == "all" else
                                                       (ops.NORM_HEAD_BEFORE if self.norm_first else ops.NORM_HEAD_AFTER))
        ops.rope_kv_general(proj, q, k_plane if self.own_kv else None, v_plane if self.own_kv else None, block_table,
                            ctx.cache.block_tokens, ctx.token_seq, ctx.token_pos, ctx.slot_ids, epilogue.inv_freq, epilogue.rope_dim,
                            self.q_gain, self.k_gain, mode, self.eps, nh, nkv, d, dv, self.own_kv)
        out = torch.empty((T, nh * dv), dtype=q.dtype, device=q.device)
        if not fast.try_attention_kv(out, q, k_plane, v_plane, block_table, ctx, nh, nkv, d, dv, self.scale, self.window, self.sink):
            split, max_splits, acc, ml = 0, 0, None, None
            if ctx.decode and ctx.max_kv_len > SPLIT_KEYS:
                split = SPLIT_KEYS
                max_splits = -(-ctx.max_kv_len // SPLIT_KEYS)
                na, nm = ops.attention_simt_scratch(T, nh, dv, max_splits)
                acc = torch.empty(na, dtype=torch.float32, device=out.device)
                ml = torch.empty(nm, dtype=torch.float32, device=out.device)
            ops.attention_simt_kv(out, q, k_plane, v_plane, block_table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs,
                                  ctx.max_new_tokens, nh, nkv, d, dv, self.scale, self.window, self.sink, split, max_splits, acc, ml)
        if gate is not None:
            ops.sigmoid_gate(out, gate, nh, dv, True)
        if store:
            self.out_store(out, out=residual)
        else:
            self.out.add_then_norm(out, residual, getattr(ctx, "norm_ahead", None), ctx)

    def attend(self, out, q, k_plane, v_plane, block_table, ctx) -> None:
        from ..kernels import fast
        nh, nkv, d = self.heads, self.kv_heads, self.head_dim
        if fast.try_attention(out, q, k_plane, v_plane, block_table, ctx, nh, nkv, d, self.scale, self.window):
            return
        split, max_splits, acc, ml = 0, 0, None, None
        if ctx.decode and ctx.max_kv_len > SPLIT_KEYS:
            split = SPLIT_KEYS
            max_splits = -(-ctx.max_kv_len // SPLIT_KEYS)
            na, nm = ops.attention_simt_scratch(ctx.num_tokens, nh, d, max_splits)
            acc = torch.empty(na, dtype=torch.float32, device=out.device)
            ml = torch.empty(nm, dtype=torch.float32, device=out.device)
        ops.attention_simt(out, q, k_plane, v_plane, block_table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens,
                           ctx.num_seqs, ctx.max_new_tokens, nh, nkv, d, self.scale, self.window, split,
                           max_splits, acc, ml)


register_part("mixer", "gqa_attention", GQAAttention)
