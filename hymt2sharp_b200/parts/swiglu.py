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


class ClampedGLU:
    """A gated feed-forward with biases and clamps:

        g = min(W_gate x + b_gate, limit);  u = clamp(W_up x + b_up, -limit, limit);  y = g * sigmoid(alpha * g) * (u + 1);  out = W_down y + b_down

    Gate and up are one product over the stacked weight; a small kernel adds the biases, clamps and applies the activation
    (float32 arithmetic); the output bias is added behind the down product."""
    graph_safe = True
    can_store = True

    def __init__(self, hidden: int, intermediate: int, limit: float, alpha: float, gate_proj: str, up_proj: str, down_proj: str,
                 gate_bias: str | None = None, up_bias: str | None = None, down_bias: str | None = None):
        if (gate_bias is None) != (up_bias is None):
            raise ValueError("the gate's and the up projection's biases come together or not at all")
        if not limit > 0:
            raise ValueError(f"a clamp at {limit}: the limit must be positive")
        self.hidden, self.intermediate, self.limit, self.alpha = int(hidden), int(intermediate), float(limit), float(alpha)
        self.names = dict(g=gate_proj, u=up_proj, d=down_proj, gb=gate_bias, ub=up_bias, db=down_bias)
        self.gate_up = self.down = self.down_store = self.bias_in = self.bias_out = None

    def tensors(self):
        h, f, n = self.hidden, self.intermediate, self.names
        t = {n["g"]: TensorSpec((f, h)), n["u"]: TensorSpec((f, h)), n["d"]: TensorSpec((h, f))}
        if n["gb"] is not None:
            t[n["gb"]] = TensorSpec((f,))
            t[n["ub"]] = TensorSpec((f,))
        if n["db"] is not None:
            t[n["db"]] = TensorSpec((h,))
        return t

    def load(self, weights, device, dtype):
        n = self.names
        self.gate_up = Linear(compute_form(torch.cat([weights[n["g"]], weights[n["u"]]], dim=0), device, dtype), role="gate_up")
        self.down = Linear(compute_form(weights[n["d"]], device, dtype), ops.EPILOGUE_ACCUMULATE, role="down")
        self.down_store = Linear(self.down.weight, ops.EPILOGUE_STORE, role="down")
        if n["gb"] is not None:
            self.bias_in = torch.cat([weights[n["gb"]], weights[n["ub"]]]).to(device).float().contiguous()
        if n["db"] is not None:
            self.bias_out = weights[n["db"]].to(device).float().contiguous()

    def first_weights(self):
        return self.gate_up.weight if self.gate_up is not None else None

    def forward(self, x, residual: torch.Tensor, ctx, store: bool = False) -> None:
        both = self.gate_up(x, ctx=ctx)
        act = torch.empty((both.shape[0], self.intermediate), dtype=both.dtype, device=both.device)
        ops.clamped_glu(act, both, self.bias_in, self.limit, self.alpha)
        ctx.prenormed = None
        if store:
            self.down_store(act, out=residual)
        else:
            self.down(act, out=residual)
        if self.bias_out is not None:
            ops.bias_act(residual, self.bias_out, 0)


register_part("feed_forward", "clamped_glu", ClampedGLU)
