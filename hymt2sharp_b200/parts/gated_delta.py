"""The gated delta rule as a mixer part: a recurrence over a matrix of state per head with a decay per key channel and a write
that first takes away what the state already answers for the key.

q = W_q x and k = W_k x (kv_heads x dim), v = W_v x (heads x vdim), no biases; value head h uses q/k head h // (heads / kv_heads).
Each of q, k, v passes a short causal convolution over time on every channel and then SiLU.  q and k become unit vectors per
head, x / sqrt(sum(x^2) + unit_eps), q also times dim^(-1/2).  beta = sigmoid(W_b x), one per head.  One decay per head and key
channel, g = exp(-exp(A_log[h]) * softplus(W_a2 (W_a1 x) + dt_bias)), laid out heads x dim.  Per head, with S [dim, vdim] from
zero:

    S <- diag(g_t) S;   u = beta_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t

Each head's o is divided by its root mean square over vdim (eps), times a stored gain of vdim entries that the heads share,
times sigmoid(W_g2 (W_g1 x)) laid out heads x vdim; then W_o.  S (float32) and the convolutions' last inputs are the
sequence's state.  Everything that enters the recurrence behind the convolutions is float32: the unit vectors, beta, the
decays (their inner product W_a2 (.) leaves the product kernel in float32), the state, o and its norm.
One product makes q, k, v and the inner vectors of the decay and the gate (a1, g1 rows); beta's product leaves its kernel in
float32; one convolution runs over q, k, v side by side.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import MixerSlot, register_part
from .conv import ShortConv
from .linear import Linear, compute_form

UNIT_EPS = 1e-6   # inside the root of the unit vectors' length


class GatedDelta:
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, heads: int, kv_heads: int, dim: int, vdim: int, taps: int, eps: float, q_proj: str, k_proj: str,
                 v_proj: str, q_conv: str, k_conv: str, v_conv: str, b_proj: str, a_log: str, a1_proj: str, a2_proj: str, dt_bias: str,
                 g1_proj: str, g2_proj: str, norm: str, o_proj: str, decay_rank: int = -1, gate_rank: int = -1):
        if heads % kv_heads:
            raise ValueError(f"{heads} heads are not a multiple of {kv_heads} q/k heads")
        self.hidden, self.heads, self.kv_heads, self.dim, self.vdim = int(hidden), int(heads), int(kv_heads), int(dim), int(vdim)
        self.taps, self.eps, self.decay_rank, self.gate_rank = int(taps), float(eps), int(decay_rank), int(gate_rank)
        self.names = dict(q=q_proj, k=k_proj, v=v_proj, b=b_proj, A=a_log, a1=a1_proj, a2=a2_proj, dt=dt_bias, g1=g1_proj, g2=g2_proj,
                          norm=norm, o=o_proj)
        self.qkv_cols = 2 * self.kv_heads * self.dim + self.heads * self.vdim
        self.conv = ShortConv(self.qkv_cols, self.taps, [(q_conv, self.kv_heads * self.dim), (k_conv, self.kv_heads * self.dim),
                                                         (v_conv, self.heads * self.vdim)], activation="silu")
        self.proj = self.a2 = self.g2 = self.out = self.out_store = self.a_log = self.dt_bias = self.gain = None

    def tensors(self):
        n, W, kd, vd, hd = self.names, self.hidden, self.kv_heads * self.dim, self.heads * self.vdim, self.heads * self.dim
        t = {n["q"]: TensorSpec((kd, W)), n["k"]: TensorSpec((kd, W)), n["v"]: TensorSpec((vd, W)), n["b"]: TensorSpec((self.heads, W)),
             n["A"]: TensorSpec((self.heads,)), n["a1"]: TensorSpec((self.decay_rank, W)), n["a2"]: TensorSpec((hd, self.decay_rank)),
             n["dt"]: TensorSpec((hd,)), n["g1"]: TensorSpec((self.gate_rank, W)), n["g2"]: TensorSpec((vd, self.gate_rank)),
             n["norm"]: TensorSpec((self.vdim,), init="gain"), n["o"]: TensorSpec((W, vd))}
        t.update(self.conv.tensors())
        return t

    def cache_need(self):
        return None

    def _matrix_bytes(self) -> int:
        return 4 * self.heads * self.dim * self.vdim

    def state_bytes(self) -> int:
        return self._matrix_bytes() + self.conv.state_bytes()

    def load(self, weights, device, dtype):
        n = self.names
        if self.dim > ops.delta_scan_max_dk():
            raise ValueError(f"{self.dim} key channels a head: the recurrence's kernel takes up to {ops.delta_scan_max_dk()}")
        self.ra, self.rg = weights[n["a1"]].shape[0], weights[n["g1"]].shape[0]
        pad = (-(self.qkv_cols + self.ra + self.rg)) % 8
        rows = [weights[n["q"]], weights[n["k"]], weights[n["v"]], weights[n["a1"]], weights[n["g1"]]]
        if pad:   # rows of zeros, so that a token's projection is a whole number of 16-byte pieces
            rows.append(torch.zeros((pad, self.hidden), dtype=rows[0].dtype))
        self.proj = Linear(compute_form(torch.cat(rows, dim=0), device, dtype), role="qkv_small")
        self.a2 = Linear(compute_form(weights[n["a2"]], device, dtype), role="decay_out")
        self.g2 = Linear(compute_form(weights[n["g2"]], device, dtype), role="gate_out")
        self.b = Linear(compute_form(weights[n["b"]], device, dtype), role="beta")
        self.out = Linear(compute_form(weights[n["o"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="o_proj")
        self.out_store = Linear(self.out.weight, ops.EPILOGUE_STORE, role="o_proj")
        self.a_log = weights[n["A"]].to(device).float().contiguous()
        self.dt_bias = weights[n["dt"]].to(device).float().contiguous()
        self.gain = weights[n["norm"]].to(device).float().repeat(self.heads).contiguous()     # the heads share it
        self.conv.load(weights, device, dtype)

    def first_weights(self):
        return self.proj.weight if self.proj is not None else None

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, slot: MixerSlot, store: bool = False) -> None:
        T, H, G, d, dv = ctx.num_tokens, self.heads, self.kv_heads, self.dim, self.vdim
        kd, c0 = G * d, self.qkv_cols
        proj = self.proj(x, ctx=ctx)                                  # [T, q | k | v | a1 | g1]
        # the convolutions' last inputs lie behind the matrix of state in this mixer's state bytes
        conv_slot = MixerSlot(state_offset=slot.state_offset + self._matrix_bytes(), state_bytes=self.conv.state_bytes())
        qkv = self.conv.forward(proj[:, :c0], ctx, conv_slot)
        decay = self.a2(proj[:, c0:c0 + self.ra], out_dtype=torch.float32)                 # float32 sums, never rounded
        gate = self.g2(proj[:, c0 + self.ra:c0 + self.ra + self.rg])
        beta = self.b(x, out_dtype=torch.float32)
        qn = torch.empty((T, kd), dtype=torch.float32, device=proj.device)
        kn = torch.empty((T, kd), dtype=torch.float32, device=proj.device)
        ops.delta_prep(qkv[:, :2 * kd], qn, kn, decay, beta, self.dt_bias, self.a_log, H, G, d, d ** -0.5, UNIT_EPS)
        o = torch.empty((T, H * dv), dtype=torch.float32, device=proj.device)
        ops.delta_scan(o, qn, kn, decay, beta, qkv[:, 2 * kd:], ctx.cache.state, slot.state_offset, ctx.cu_seqlens, ctx.slot_ids,
                       ctx.kv_lens, ctx.num_seqs, H, G, d, dv, ctx.max_new_tokens)
        gated = torch.empty((T, H * dv), dtype=proj.dtype, device=proj.device)
        ops.head_norm_gate(gated, o, gate, self.gain, H, dv, self.eps, gate_act="sigmoid")
        if store:
            self.out_store(gated, out=residual)
            ctx.prenormed = None
        else:
            self.out.add_then_norm(gated, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("mixer", "gated_delta", GatedDelta)
