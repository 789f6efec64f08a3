"""Dense SwiGLU feed-forward: residual += (silu(x·Wg^T) * (x·Wu^T)) · Wd^T
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:27-34, src/HyMT2Sharp/Ops.cs:1053).
Gate and up are one product over the stacked weight [2F, H] whose epilogue applies
the activation, so the [T, 2F] intermediate never reaches memory.

`activation` "gelu_tanh" puts the tanh form of GELU in SiLU's place: residual += (gelu_tanh(x·Wg^T) * (x·Wu^T)) · Wd^T.
The product's epilogue knows SiLU only, so that form stores gate and up side by side and a small kernel follows."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import Linear, compute_form


ACTIVATIONS = {"silu": ops.GATED_SILU, "gelu_tanh": ops.GATED_GELU_TANH}


class SwiGLU:
    graph_safe = True  # its forward only launches kernels on the current stream
    takes_prenormed = True  # x may be a parts.base.Prenormed: the gate/up product applies the norm's row scale itself
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, intermediate: int, gate_proj: str, up_proj: str, down_proj: str, activation: str = "silu"):
        if activation not in ACTIVATIONS:
            raise ValueError(f"activation '{activation}' is not known (known: {', '.join(ACTIVATIONS)})")
        self.hidden, self.intermediate, self.activation = int(hidden), int(intermediate), activation
        self.names = dict(g=gate_proj, u=up_proj, d=down_proj)
        self.gate_up = self.down = None

    def tensors(self):
        h, f, n = self.hidden, self.intermediate, self.names
        return {n["g"]: TensorSpec((f, h)), n["u"]: TensorSpec((f, h)), n["d"]: TensorSpec((h, f))}

    def load(self, weights, device, dtype):
        n = self.names
        stacked = torch.cat([weights[n["g"]], weights[n["u"]]], dim=0)
        fused = self.activation == "silu"
        self.gate_up = Linear(compute_form(stacked, device, dtype), ops.EPILOGUE_SWIGLU if fused else ops.EPILOGUE_STORE, role="gate_up")
        self.down = Linear(compute_form(weights[n["d"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="down")
        self.down_store = Linear(self.down.weight, ops.EPILOGUE_STORE, role="down")

    def first_weights(self):
        """The weights that this part's first kernel streams."""
        return self.gate_up.weight if self.gate_up is not None else None

    def forward(self, x, residual: torch.Tensor, ctx, store: bool = False) -> None:
        act = self.gate_up(x, ctx=ctx)
        if self.activation != "silu":
            both, act = act, torch.empty((act.shape[0], self.intermediate), dtype=act.dtype, device=act.device)
            ops.gated_act(act, both, ACTIVATIONS[self.activation])
        if store:
            self.down_store(act, out=residual)
            ctx.prenormed = None
        else:
            self.down.add_then_norm(act, residual, getattr(ctx, "norm_ahead", None), ctx)


register_part("feed_forward", "swiglu", SwiGLU)
