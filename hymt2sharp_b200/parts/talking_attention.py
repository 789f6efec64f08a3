"""Softmax attention whose heads talk, over the paged cache, as a mixer part.

q = W_q x (heads x dim), k = W_k x (kv_heads x dim), no biases; optionally a short causal convolution over time on every
channel of q and k directly behind the projections (its last inputs are state of the sequence); the VALUES are the keys as
they stand in front of the rotation (`values="keys"`, no value projection).  Then rotary positions on q and k, and

    raw_g(i, j) = (q_g(i) . k_g(j)) * scale * temp[g]            temp: a stored number per head
    s_h(i, j)   = sum_g talk[h, g] raw_g(i, j)                   talk: a stored [heads, heads] matrix
    p_h(i, j)   = exp(s_h(i, j)) / (exp(sink_h) + sum_j' exp(s_h(i, j')))      sink: a stored number per head (or none)

over the keys that i sees: j <= i, and with `mask` "chunk" only those of i's own chunk of `mask_size` positions (chunks are
counted from position 0 of the sequence, however the prompt was cut into steps), with "window" only the last `mask_size`.
Head h reads key/value head h // (heads / kv_heads).  The heads side by side are multiplied entry by entry by
sigmoid(W_g x) (`g_proj`, optional) and projected by W_o.  Scores, the mixing, the softmax and the angles are float32.

A chunk never reaches back further than its size, so the cache keeps this mixer's keys in a window group of that size and
gives older blocks back.  One product makes q, k and the gate's input; one convolution runs over q and k side by side.
"""
from __future__ import annotations

import torch

from ..cache.allocator import GroupSpec
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, PartSpec, build_part, register_part
from .conv import ShortConv
from .linear import Linear, compute_form


class TalkingAttention:
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, scale: float, position: PartSpec | None, q_proj: str, k_proj: str,
                 o_proj: str, talk: str, temp: str, sink: str | None = None, g_proj: str | None = None, mask: str | None = None,
                 mask_size: int = 0, taps: int = 0, q_conv: str | None = None, k_conv: str | None = None, values: str = "keys"):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} kv heads")
        if values != "keys":
            raise ValueError(f"values '{values}': this attention takes its values from its keys ('keys')")
        if mask not in (None, "chunk", "window") or (mask is not None and mask_size < 1):
            raise ValueError(f"mask '{mask}' of size {mask_size}: known are 'chunk', 'window' (with a size of at least 1) and None")
        if taps and (q_conv is None or k_conv is None):
            raise ValueError("a convolution on q and k needs the names of both filters")
        self.hidden, self.heads, self.kv_heads, self.dim, self.scale = int(hidden), int(heads), int(kv_heads), int(dim), float(scale)
        self.mask, self.mask_size = mask, int(mask_size) if mask is not None else 0
        self.names = dict(q=q_proj, k=k_proj, o=o_proj, g=g_proj, talk=talk, temp=temp, sink=sink)
        self.position = build_part("position", position) if position is not None else None
        qk = (self.heads + self.kv_heads) * self.dim
        self.conv = ShortConv(qk, taps, [(q_conv, self.heads * self.dim), (k_conv, self.kv_heads * self.dim)]) if taps else None
        self.proj = self.out = self.out_store = self.talk = self.temp = self.sink = None

    def tensors(self):
        n, H, qd, kd = self.names, self.heads, self.heads * self.dim, self.kv_heads * self.dim
        t = {n["q"]: TensorSpec((qd, self.hidden)), n["k"]: TensorSpec((kd, self.hidden)), n["o"]: TensorSpec((self.hidden, qd)),
             n["talk"]: TensorSpec((H, H), init="identity"), n["temp"]: TensorSpec((H,), init="gain")}
        if n["sink"] is not None:
            t[n["sink"]] = TensorSpec((H,))
        if n["g"] is not None:
            t[n["g"]] = TensorSpec((qd, self.hidden))
        if self.conv is not None:
            t.update(self.conv.tensors())
        if self.position is not None:
            t.update(self.position.tensors())
        return t

    def cache_need(self):
        if self.mask is None:
            return GroupSpec("full", self.kv_heads, self.dim, planes=0)
        return GroupSpec("window", self.kv_heads, self.dim, planes=0, window=self.mask_size)

    def state_bytes(self) -> int:
        return self.conv.state_bytes() if self.conv is not None else 0

    def load(self, weights, device, dtype):
        n = self.names
        rows = [weights[n["q"]], weights[n["k"]]] + ([weights[n["g"]]] if n["g"] is not None else [])
        self.proj = Linear(compute_form(torch.cat(rows, dim=0), device, dtype), role="qkg")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        self.talk = weights[n["talk"]].to(device).float().contiguous()
        self.temp = weights[n["temp"]].to(device).float().contiguous()
        self.sink = weights[n["sink"]].to(device).float().contiguous() if n["sink"] is not None else None
        if self.conv is not None:
            self.conv.load(weights, device, dtype)
        if self.position is not None:
            self.position.load(weights, device, dtype)

    def first_weights(self):
        return self.proj.weight if self.proj is not None else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, H, G, d = ctx.num_tokens, self.heads, self.kv_heads, self.dim
        qk = (H + G) * d
        rotary = self.position.kernel_epilogue(ctx) if self.position is not None else None
        if rotary is not None and rotary.rope_dim and (rotary.pairing != "interleaved" or rotary.amplitude != 1.0):
            raise ValueError("this attention rotates neighbouring pairs by a table of frequencies; its position encoding must offer that form")
        proj = self.proj(x, ctx=ctx)                                  # [T, q | k | gate input]
        rows = proj[:, :qk]
        if self.conv is not None:
            rows = self.conv.forward(rows, ctx, slot)                  # the convolution's state is this mixer's state
        k_plane, v_plane = ctx.cache.plane(slot.group, slot.plane)
        table = ctx.cache.tables[slot.group]
        q = torch.empty((T, H * d), dtype=proj.dtype, device=proj.device)
        ops.talk_prep(rows, q, k_plane if slot.writes else None, v_plane if slot.writes else None, table, ctx.cache.block_tokens,
                      ctx.token_seq, ctx.token_pos, ctx.slot_ids, rotary.inv_freq if rotary else None, rotary.rope_dim if rotary else 0,
                      H, G, d)
        out = torch.empty((T, H * d), dtype=proj.dtype, device=proj.device)
        gate = proj[:, qk:qk + H * d] if self.names["g"] is not None else None
        ops.talking_attention(out, q, gate, k_plane, v_plane, table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs,
                              ctx.max_new_tokens, H, G, d, self.scale, self.talk, self.temp, self.sink, self.mask, self.mask_size,
                              max_kv_len=ctx.max_kv_len)
        if store:
            self.out_store(out, out=residual)
            ctx.prenormed = None
        else:
            self.out.add_then_norm(out, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("mixer", "talking_attention", TalkingAttention)
