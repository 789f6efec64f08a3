"""Time mixing with a decay per token and channel (in the manner of RWKV's sixth generation), as a mixer part.

With x' the token before (zeros in front of a sequence's first token), each of r, k, v, g, w reads its own mixture
m_s = x + (x' - x) * mu_s.  r, k, v = W_r m_r, W_k m_k, W_v m_v (heads x dim), gate = silu(W_g m_g); the decay is

    w = exp(-exp(W_w2 tanh(W_w1 m_w) + w0))        per head and key channel, in (0, 1)

and per head, with S [dim, dim] starting at zero and the bonus u for the current token only,

    o_t = (S_(t-1) + diag(u) k_t v_t^T)^T r_t,      S_t = diag(w_t) S_(t-1) + k_t v_t^T.

Each head's o is divided by its root mean square, the heads side by side are multiplied by a stored gain and by the gate,
and projected by W_o.  S and the last x of the step before are the sequence's state (float32, in the cache's state row).
The decay with everything inside it, the recurrence, the state and the norm are float32; the projections have the
engine's compute type.  The width of the decay's inner projection is the checkpoint's (`decay_rank`; None: whatever W_w1
holds).
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, register_part
from .linear import Linear, compute_form, matmul, matmul_batched
from .state_scan import chunk_plan

MIXES = "rkvgw"   # the order of the mixtures in one row of the shifted input


class TimeMix:
    graph_safe = True
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, heads: int, dim: int, eps: float, mu: str, r_proj: str, k_proj: str, v_proj: str, g_proj: str,
                 w1_proj: str, w2_proj: str, w0: str, bonus: str, norm: str, o_proj: str, decay_rank: int | None = None):
        """`mu`: the tensor names of the five mixing vectors with `{}` in place of r, k, v, g, w."""
        self.hidden, self.heads, self.dim, self.eps = int(hidden), int(heads), int(dim), float(eps)
        self.decay_rank = int(decay_rank) if decay_rank else None
        self.names = dict(mu=mu, r=r_proj, k=k_proj, v=v_proj, g=g_proj, w1=w1_proj, w2=w2_proj, w0=w0, u=bonus, n=norm, o=o_proj)
        self.mu = self.rkvg = self.w1 = self.w2 = self.w0 = self.u = self.gain = self.out = self.out_store = None

    def tensors(self):
        n, h, D = self.names, self.hidden, self.heads * self.dim
        rank = self.decay_rank or -1     # -1: any size, the checkpoint's
        t = {n["mu"].format(s): TensorSpec((h,)) for s in MIXES}
        t.update({n[s]: TensorSpec((D, h)) for s in "rkvg"})
        t.update({n["w1"]: TensorSpec((rank, h)), n["w2"]: TensorSpec((D, rank)), n["w0"]: TensorSpec((D,)),
                  n["u"]: TensorSpec((self.heads, self.dim)), n["n"]: TensorSpec((D,), init="gain"), n["o"]: TensorSpec((h, D))})
        return t

    def cache_need(self):
        return None

    def state_bytes(self) -> int:
        # S float32 [heads, dim, dim], then the last input row float32 [hidden]
        return 4 * self.heads * self.dim * self.dim + 4 * self.hidden

    def load(self, weights, device, dtype):
        n = self.names
        small = lambda name: weights[name].to(device).float().reshape(-1).contiguous()
        if weights[n["w1"]].shape[0] != weights[n["w2"]].shape[1]:
            raise ValueError(f"{n['w1']} makes {weights[n['w1']].shape[0]} entries, {n['w2']} reads {weights[n['w2']].shape[1]}")
        self.mu = torch.stack([small(n["mu"].format(s)) for s in MIXES]).contiguous()
        self.rkvg = compute_form(torch.stack([weights[n[s]] for s in "rkvg"]), device, dtype)
        self.w1 = Linear(compute_form(weights[n["w1"]], device, dtype), role="decay_in")
        # the decay's outer projection reads float32 (tanh of float32 sums) and is small: float32 weights, CUDA cores
        self.w2 = weights[n["w2"]].to(device).float().contiguous()
        self.w0, self.u, self.gain = small(n["w0"]), small(n["u"]), small(n["n"])
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")

    def first_weights(self):
        return self.rkvg

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, H, D = ctx.num_tokens, self.hidden, self.heads * self.dim
        state_s = 4 * self.heads * self.dim * self.dim
        mixes = torch.empty((T, len(MIXES) * H), dtype=x.dtype, device=x.device)
        ops.token_shift(mixes, x, self.mu, ctx.cache.state, slot.state_offset + state_s, ctx.token_seq, ctx.cu_seqlens, ctx.slot_ids,
                        ctx.kv_lens)
        rkvg = torch.empty((T, 4 * D), dtype=x.dtype, device=x.device)
        ops.tag = "rkvg"
        matmul_batched(rkvg, mixes, self.rkvg, H, D)
        ops.tag = None
        inner = self.w1(mixes[:, 4 * H:], out_dtype=torch.float32)
        ops.tanh_(inner)
        xw = torch.empty((T, D), dtype=torch.float32, device=x.device)
        ops.tag = "decay_out"
        ops.gemm_simt(xw, inner, self.w2)
        ops.tag = None
        o = torch.empty((T, D), dtype=torch.float32, device=x.device)
        ops.linear_scan(o, rkvg[:, :D], rkvg[:, D:2 * D], rkvg[:, 2 * D:3 * D], ops.SCAN_TOKEN_DECAY, ctx.cache.state, slot.state_offset,
                        ctx.cu_seqlens, ctx.slot_ids, ctx.kv_lens, ctx.num_seqs, self.heads, self.dim, self.dim, x=xw, w0=self.w0,
                        u=self.u, chunks=chunk_plan(ctx))
        gated = torch.empty((T, D), dtype=x.dtype, device=x.device)
        ops.head_norm_gate(gated, o, rkvg[:, 3 * D:], self.gain, self.heads, self.dim, self.eps)
        if store:
            self.out_store(gated, out=residual)
            ctx.prenormed = None
        else:
            self.out.add_then_norm(gated, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("mixer", "time_mix", TimeMix)
