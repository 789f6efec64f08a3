"""Latent (low-rank key/value) attention over the paged cache, as a mixer part.

Per token the cache holds ONE row for all heads: the latent vector c (`kv_rank` entries, RMS-normed with a gain) and one
rotated key part (`rot_dim` entries) that every head shares.  Head h's key is [W_uk[h] c, rotated part], its value
W_uv[h] c.  Nothing per head is ever stored or rebuilt: the up-projections are moved to the other side of the products,

    score_h(t, s) = ( (W_uk[h]^T q_h[:dim]) . c_s  +  rot(q_h[dim:]) . rot(k_s) ) * scale
    out_h(t)      = W_uv[h] ( sum_s softmax_s(score_h(t, .)) c_s )

so the attention runs in the compressed space, with a query of kv_rank + rot_dim entries per head against the cached
row, whose first kv_rank entries are also the value.  Then an output gate (sigmoid of a projection of the mixer's
input, one value per output entry or one per head) and the output projection.  Scores, softmax, the latent norm and
the rotation are float32; the projections run in the engine's compute type.

A prompt that starts at position 0 brings all of its keys along, and a head's own rows (dim + rot_dim, vdim) are several
times narrower than the compressed row: there the bfloat16 engine rebuilds every head's keys and values with one product
over all tokens and runs the attention per head, which is the same sums in another order (EXPAND_FROM_TOKENS).

`own_kv` False: the layer has no down-projection and no latent norm; it attends over the compressed rows that another run
cached (the model's order names it), with its own up-projections, queries, window and gate.  `cache_window`: the positions that
the cache keeps for this plane when that is more than the layer's own window (readers of one plane may look back differently
far; 0 with a window elsewhere means: keep everything).
"""
from __future__ import annotations

import torch

from ..cache.allocator import GroupSpec
from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, PartSpec, build_part, register_part
from .linear import Linear, compute_form, matmul_batched

EXPAND_FROM_TOKENS = 32   # prompts from this length on are worth one more product (keys and values per head)
SPLIT_KEYS = 256     # decode: keys per partial, a constant so that the cut depends on nothing else
SPLIT_KEYS_TC = 128  # the same for the tensor-core kernel, whose blocks are few and large: two tiles of keys each (one tile each
                     # measured slower: twice the partials to write and fold)


class LatentAttention:
    graph_safe = True  # its forward only launches kernels on the current stream
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, heads: int, dim: int, rot_dim: int, vdim: int, kv_rank: int, scale: float, eps: float,
                 position: PartSpec | None, gate: str | None, q_proj: str, dkv_proj: str, dkv_norm: str, uk_proj: str,
                 uv_proj: str, o_proj: str, g_proj: str | None = None, window: int | None = None, own_kv: bool = True,
                 cache_window: int | None = None):
        if gate not in (None, "element", "head"):
            raise ValueError(f"output gate '{gate}': known are 'element' (one value per output entry), 'head' and None")
        if gate is not None and g_proj is None:
            raise ValueError("an output gate needs its projection's tensor name")
        self.hidden, self.heads, self.dim, self.rot, self.vdim, self.rank = hidden, heads, dim, rot_dim, vdim, kv_rank
        self.scale, self.eps, self.gate, self.window = float(scale), float(eps), gate, int(window or 0)
        self.own_kv = bool(own_kv)
        self.cache_window = self.window if cache_window is None else int(cache_window)
        if self.cache_window and (not self.window or self.cache_window < self.window):
            raise ValueError(f"a cache that keeps {self.cache_window} positions is too short for a window of {self.window or 'everything'}")
        self.names = dict(q=q_proj, dkv=dkv_proj, cn=dkv_norm, uk=uk_proj, uv=uv_proj, o=o_proj, g=g_proj)
        self.position = build_part("position", position) if position is not None else None
        self.q_cols = heads * (dim + rot_dim)
        self.gate_cols = 0 if gate is None else (heads * vdim if gate == "element" else heads)
        self.proj = self.out = self.uk_t = self.uv = self.c_gain = self.ukv = None

    # -- what it needs ----------------------------------------------------------
    def tensors(self):
        n, H = self.names, self.heads
        t = {n["q"]: TensorSpec((self.q_cols, self.hidden)), n["uk"]: TensorSpec((H * self.dim, self.rank)),
             n["uv"]: TensorSpec((H * self.vdim, self.rank)), n["o"]: TensorSpec((self.hidden, H * self.vdim))}
        if self.own_kv:
            t[n["dkv"]] = TensorSpec((self.rank + self.rot, self.hidden))
            t[n["cn"]] = TensorSpec((self.rank,), init="gain")
        if self.gate is not None:
            t[n["g"]] = TensorSpec((self.gate_cols, self.hidden))
        if self.position is not None:
            t.update(self.position.tensors())
        return t

    def cache_need(self):
        kind = "window" if self.cache_window > 0 else "full"
        return GroupSpec(kind, 1, self.rank + self.rot, planes=0, window=self.cache_window, streams=1)

    def state_bytes(self) -> int:
        return 0

    def load(self, weights, device, dtype):
        n, H = self.names, self.heads
        rows = [weights[n["q"]]] + ([weights[n["dkv"]]] if self.own_kv else []) + ([weights[n["g"]]] if self.gate is not None else [])
        total = sum(r.shape[0] for r in rows)
        if total % 8:
            # rows of zeros, so that a token's projection is a whole number of 16-byte pieces and kernels may read it by them
            rows.append(torch.zeros((8 - total % 8, self.hidden), dtype=rows[0].dtype))
        self.proj = Linear(compute_form(torch.cat(rows, dim=0), device, dtype), role="q_dkv_gate")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        # per head: W_uk[h]^T [kv_rank, dim] (the query goes into the compressed space) and W_uv[h] [vdim, kv_rank]
        uk = weights[n["uk"]].reshape(H, self.dim, self.rank).transpose(1, 2)
        self.uk_t = compute_form(uk, device, dtype)
        self.uv = compute_form(weights[n["uv"]].reshape(H, self.vdim, self.rank), device, dtype)
        self.c_gain = weights[n["cn"]].to(device).float().contiguous() if self.own_kv else torch.ones(self.rank, dtype=torch.float32, device=device)
        if self.rank % 8 == 0 and ops.latent_attention_expanded_supported(dtype, self.dim, self.rot, self.vdim):
            # every head's key and value rows in one product over the latent vectors: [W_uk; W_uv]
            self.ukv = Linear(compute_form(torch.cat([weights[n["uk"]], weights[n["uv"]]], dim=0), device, dtype), role="kv_expand")
        if self.position is not None:
            self.position.load(weights, device, dtype)

    # -- the step ---------------------------------------------------------------
    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, H, dl = ctx.num_tokens, self.heads, self.rank + self.rot
        rotary = self.position.kernel_epilogue(ctx) if self.position is not None else None
        if rotary is not None and rotary.rope_dim and rotary.pairing != "interleaved":
            raise ValueError("latent attention rotates neighbouring pairs; its position encoding must offer that form")
        plane, _ = ctx.cache.plane(slot.group, slot.plane)
        table = ctx.cache.tables[slot.group]
        if slot.writes != self.own_kv:
            raise ValueError("a latent attention without a down-projection reads another run's cache plane, and only such a one does")
        proj = self.proj(x, ctx=ctx)                                   # [T, queries | latent row (if its own) | gate]
        kept = ("latent_rows", slot.group, slot.plane)                 # a step's compressed rows side by side, for the plane's readers
        if (self.ukv is not None and not ctx.decode and ctx.max_new_tokens >= EXPAND_FROM_TOKENS and ctx.host_starts
                and not any(ctx.host_starts) and (self.own_kv or kept in ctx.shared)):
            out = self._attend_expanded(proj, rotary, plane if slot.writes else None, table, ctx, kept)
            self._gate_and_project(out, proj, residual, ctx, store)
            return
        q = torch.empty((T, H * dl), dtype=proj.dtype, device=proj.device)
        ops.latent_prep(proj, self.q_cols, q, plane if slot.writes else None, table, ctx.cache.block_tokens, ctx.token_seq,
                        ctx.token_pos, ctx.slot_ids, self.c_gain, rotary.inv_freq if rotary else None,
                        rotary.rope_dim if rotary else 0, rotary.amplitude if rotary else 1.0, self.eps, H, self.dim,
                        self.rot, self.rank)
        # q[t, h, :kv_rank] = W_uk[h]^T q_h[:dim]
        ops.tag = "q_absorb"
        matmul_batched(q, proj, self.uk_t, self.dim + self.rot, dl)
        ops.tag = None
        mixed = torch.empty((T, H * self.rank), dtype=q.dtype, device=q.device)
        self.attend(mixed, q, plane, table, ctx)
        out = torch.empty((T, H * self.vdim), dtype=q.dtype, device=q.device)
        ops.tag = "v_up"
        matmul_batched(out, mixed, self.uv, self.rank, self.vdim)
        ops.tag = None
        self._gate_and_project(out, proj, residual, ctx, store)

    def _gate_and_project(self, out, proj, residual, ctx, store: bool) -> None:
        if self.gate is not None:
            g0 = self.q_cols + (self.rank + self.rot if self.own_kv else 0)
            ops.sigmoid_gate(out, proj[:, g0:g0 + self.gate_cols], self.heads, self.vdim, self.gate == "head")
        if store:
            self.out_store(out, out=residual)
        else:
            self.out.add_then_norm(out, residual, getattr(ctx, "norm_ahead", None), ctx)

    def _attend_expanded(self, proj, rotary, plane, table, ctx, kept) -> torch.Tensor:
        """Whole prompts from position 0: the cache rows are written as always and also kept side by side (for this layer and
        for the layers that read its plane in the same step); one product makes every head's keys and values from them; the
        attention runs per head on the tensor cores."""
        T, H = ctx.num_tokens, self.heads
        if self.own_kv:
            rows = torch.empty((T, self.rank + self.rot), dtype=proj.dtype, device=proj.device)
            ctx.shared[kept] = rows
        else:
            rows = ctx.shared[kept]
        ops.latent_prep(proj, self.q_cols, None, plane, table, ctx.cache.block_tokens, ctx.token_seq, ctx.token_pos, ctx.slot_ids,
                        self.c_gain, rotary.inv_freq if rotary else None, rotary.rope_dim if rotary else 0,
                        rotary.amplitude if rotary else 1.0, self.eps, H, self.dim, self.rot, self.rank,
                        rows_out=rows if self.own_kv else None)
        kv = self.ukv(rows[:, :self.rank], ctx=ctx)                    # [T, H * dim | H * vdim]
        out = torch.empty((T, H * self.vdim), dtype=proj.dtype, device=proj.device)
        ops.latent_attention_expanded(out, proj[:, :self.q_cols], kv[:, :H * self.dim], kv[:, H * self.dim:], rows[:, self.rank:],
                                      ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs, ctx.max_new_tokens, H, self.dim,
                                      self.rot, self.vdim, self.scale, self.window)
        return out

    def attend(self, out, q, plane, table, ctx) -> None:
        # bfloat16 with rows in pieces of 16: the tensor-core kernel; 32-bit and odd sizes: the general CUDA-core kernel
        run, keys = ops.attention_shared_vector, SPLIT_KEYS
        if ops.latent_attention_mma_supported(out.dtype, self.rank + self.rot, self.rank, plane.shape[2]):
            run, keys = ops.latent_attention_mma, SPLIT_KEYS_TC
        split, max_splits, acc, ml = 0, 0, None, None
        if ctx.decode and ctx.max_kv_len > keys:
            split = keys
            max_splits = -(-ctx.max_kv_len // keys)
            acc = torch.empty(ctx.num_tokens * self.heads * max_splits * self.rank, dtype=torch.float32, device=out.device)
            ml = torch.empty(ctx.num_tokens * self.heads * max_splits * 2, dtype=torch.float32, device=out.device)
        run(out, q, plane, table, ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs, ctx.max_new_tokens, self.heads,
            self.rank + self.rot, self.rank, self.scale, self.window, split, max_splits, acc, ml)


register_part("mixer", "latent_attention", LatentAttention)
