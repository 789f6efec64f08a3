"""Short causal convolution over time, one filter per channel, with the sequence's last inputs kept as state.

out_t = [x_t +] [bias +] sum_j w[:, j] * x_(t - taps + 1 + j): the last column of w [channels, taps] multiplies the
current token, and what lies before a sequence's start counts as zero.  The last taps - 1 inputs of every sequence
are part of its state (float32 [taps - 1, channels] in the cache's state row), so a step continues where the step
before ended, however the tokens were cut into steps.  It is a helper of blocks and mixers, not a part category of
its own: whoever holds one asks `state_bytes()` and hands it the MixerSlot that the model laid out for it.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec


class ShortConv:
    graph_safe = True

    def __init__(self, channels: int, taps: int, weight, bias: str | None = None, add_input: bool = False,
                 activation: str | None = None):
        if taps < 1:
            raise ValueError(f"a convolution needs at least one tap, got {taps}")
        if activation not in (None, "silu"):
            raise ValueError(f"activation '{activation}' of a convolution: known are 'silu' and None")
        self.channels, self.taps, self.add_input, self.activation = int(channels), int(taps), bool(add_input), activation
        # `weight`: one tensor name, or [(name, channels), ...]: several filters side by side that run as one convolution
        self.pieces = [(weight, self.channels)] if isinstance(weight, str) else [(n, int(c)) for n, c in weight]
        if sum(c for _, c in self.pieces) != self.channels:
            raise ValueError("the filters side by side do not add up to the convolution's channels")
        self.weight_name, self.bias_name = self.pieces[0][0], bias
        self.w = self.b = None

    def tensors(self):
        t = {name: TensorSpec((c, self.taps)) for name, c in self.pieces}
        if self.bias_name is not None:
            t[self.bias_name] = TensorSpec((self.channels,))
        return t

    def state_bytes(self) -> int:
        return 4 * (self.taps - 1) * self.channels

    def load(self, weights, device, dtype):
        # the filter and its bias are used as float32 in both precisions (they are a few values per channel)
        self.w = torch.cat([weights[name].to(device).float() for name, _ in self.pieces], dim=0).contiguous()
        self.b = weights[self.bias_name].to(device).float().contiguous() if self.bias_name is not None else None

    def forward(self, x: torch.Tensor, ctx, slot) -> torch.Tensor:
        """x [T, channels] (rows may be columns of a wider matrix); returns a new [T, channels] of x's type."""
        out = torch.empty((x.shape[0], self.channels), dtype=x.dtype, device=x.device)
        ops.causal_conv(out, x, self.w, self.b, ctx.cache.state, slot.state_offset, ctx.cu_seqlens, ctx.slot_ids,
                        ctx.kv_lens, ctx.num_seqs, ctx.max_new_tokens, self.add_input, self.activation == "silu")
        return out
