"""Retention as a mixer part: linear attention with a fixed decay per head, no softmax and no denominator.

q = W_q x, k = W_k x * dim^(-1/2) (heads x dim), v = W_v x (heads x vdim), no biases.  Per head, with S [dim, vdim] starting
at zero:

    S_t = decay_h * S_(t-1) + k_t v_t^T,      o_t = S_t^T q_t

Each head's o is divided by its root mean square (no gain), the heads side by side are multiplied by silu(W_g x) and
projected by W_o.  With a `position` encoding the first entries of every q and k head are rotated by the token's position in
front of the recurrence (the scale of k commutes with the rotation); the rotated q and k are then handed to the recurrence in
float32, never rounded.  S is float32 and is the sequence's state, carried from step to step in the cache's state row; scores,
state and the norm are float32, the projections have the engine's compute type.  One product makes q, k, v and the gate.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, PartSpec, build_part, register_part
from .linear import Linear, compute_form
from .state_scan import chunk_plan


class Retention:
    graph_safe = True
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, heads: int, dim: int, vdim: int, decay: list, eps: float, q_proj: str, k_proj: str, v_proj: str,
                 g_proj: str, o_proj: str, position: PartSpec | None = None):
        if len(decay) != heads:
            raise ValueError(f"{len(decay)} decays for {heads} heads")
        self.hidden, self.heads, self.dim, self.vdim, self.eps = int(hidden), int(heads), int(dim), int(vdim), float(eps)
        self.decay_host = [float(d) for d in decay]
        self.names = dict(q=q_proj, k=k_proj, v=v_proj, g=g_proj, o=o_proj)
        self.position = build_part("position", position) if position is not None else None
        self.qkvg = self.out = self.out_store = self.decay = None

    def tensors(self):
        n, h, qd, vd = self.names, self.hidden, self.heads * self.dim, self.heads * self.vdim
        return {n["q"]: TensorSpec((qd, h)), n["k"]: TensorSpec((qd, h)), n["v"]: TensorSpec((vd, h)), n["g"]: TensorSpec((vd, h)),
                n["o"]: TensorSpec((h, vd))}

    def cache_need(self):
        return None

    def state_bytes(self) -> int:
        return 4 * self.heads * self.dim * self.vdim

    def load(self, weights, device, dtype):
        n = self.names
        stacked = torch.cat([weights[n[s]] for s in "qkvg"], dim=0)
        self.qkvg = Linear(compute_form(stacked, device, dtype), role="qkvg")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        self.decay = torch.tensor(self.decay_host, dtype=torch.float32, device=device)
        if self.position is not None:
            self.position.load(weights, device, dtype)

    def first_weights(self):
        return self.qkvg.weight if self.qkvg is not None else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, qd, vd = ctx.num_tokens, self.heads * self.dim, self.heads * self.vdim
        proj = self.qkvg(x, ctx=ctx)
        q, k, v, g = proj[:, :qd], proj[:, qd:2 * qd], proj[:, 2 * qd:2 * qd + vd], proj[:, 2 * qd + vd:]
        rotary = self.position.kernel_epilogue(ctx) if self.position is not None else None
        if rotary is not None and rotary.rope_dim:
            if rotary.amplitude != 1.0:
                raise ValueError("retention rotates by a table of frequencies; its position encoding scales cosine and sine")
            # q and k of all heads are 2 * heads heads side by side; v is carried along, so that the recurrence reads one type
            turned = torch.empty((T, 2 * qd + vd), dtype=torch.float32, device=proj.device)
            ops.rotate_heads(turned, proj[:, :2 * qd + vd], ctx.token_pos, rotary.inv_freq, 2 * self.heads, self.dim, rotary.rope_dim,
                             rotary.pairing)
            q, k, v = turned[:, :qd], turned[:, qd:2 * qd], turned[:, 2 * qd:]
        o = torch.empty((T, vd), dtype=torch.float32, device=proj.device)
        ops.linear_scan(o, q, k, v, ops.SCAN_FIXED_DECAY, ctx.cache.state, slot.state_offset, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens,
                        ctx.num_seqs, self.heads, self.dim, self.vdim, decay=self.decay, k_scale=self.dim ** -0.5, chunks=chunk_plan(ctx))
        gated = torch.empty((T, vd), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(gated, o, g, None, self.heads, self.vdim, self.eps)
        if store:
            self.out_store(gated, out=residual)
            ctx.prenormed = None
        else:
            self.out.add_then_norm(gated, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("mixer", "retention", Retention)
