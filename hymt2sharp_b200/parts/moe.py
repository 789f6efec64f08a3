"""A mixture of small feed-forward experts with a router: residual += sum over a token's chosen experts of weight * expert(x).

The router's outputs z = W_router x are float32 (float32 sums of the products in both engines); the scores are their
softmax over ALL outputs.  The first `experts` outputs name experts with tensors, expert(x) = W_down act(W_up x); the last
`identity` outputs name identity experts, whose output is x itself.  The `top` outputs with the largest score + correction
are chosen (`correction`: a stored vector, one entry per output; None: none); a chosen output's weight is its score, without
the correction and not renormalised.  A shared expert (any feed-forward part) runs for every token with weight 1.

Chosen by parameters beyond that: a bias of the router (`router_bias`, a stored vector added to z); weights that are the
softmax over the CHOSEN outputs only (`weights="chosen_softmax"`; the choice by score is then the choice by z); and gated
experts, expert(x) = W_down (act(W_gate x) * (W_up x)) (`gate_proj` given; act "silu"): gate and up are one grouped product
over the stacked matrices, and a small kernel applies the activation.

How a step runs: router product; `moe_route` (softmax, choice); `moe_place` sorts the (token, choice) pairs by expert, each
expert's rows padded to whole row tiles; one grouped product per projection over the sorted rows (the first gathers its
input rows by token, its epilogue is the activation); `moe_combine` adds a token's rows up in the order they were chosen.
Nothing uses atomics and every sum has a fixed order, so a token's result does not depend on the other tokens of the step.
"""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import PartSpec, build_part, register_part
from .linear import Linear, compute_form

ACTIVATIONS = {"relu2": ops.EPILOGUE_RELU_SQUARED}      # experts without a gate: an epilogue of the grouped product
GATED_ACTIVATIONS = {"silu": ops.GATED_SILU, "gelu_tanh": ops.GATED_GELU_TANH}
WEIGHTS = ("scores", "chosen_softmax")
SKINNY_MAX_PAIRS = 512        # up to this many (token, choice) pairs in a step the kernel for few rows runs the experts,
SKINNY_PAIRS_BESIDE_TC = 64   # where the tensor cores take the operands only up to this many: beyond, most experts meet several
                              # rows, and a row tile of 128 on the tensor cores, mostly empty, still reads each expert once


class RoutedExperts:
    graph_safe = True  # its forward only launches kernels on the current stream
    can_store = True   # forward(..., store=True) overwrites `residual` with its output instead of adding to it

    def __init__(self, hidden: int, experts: int, identity: int, top: int, intermediate: int, activation: str, router: str,
                 up_proj: str, down_proj: str, correction: str | None = None, shared: PartSpec | None = None,
                 gate_proj: str | None = None, router_bias: str | None = None, weights: str = "scores"):
        """`up_proj` / `down_proj` / `gate_proj`: the tensor names of expert e with `{}` in place of e."""
        known = GATED_ACTIVATIONS if gate_proj is not None else ACTIVATIONS
        if activation not in known:
            raise ValueError(f"activation '{activation}' is not known for experts {'with' if gate_proj else 'without'} a gate "
                             f"(known: {', '.join(known)})")
        if weights not in WEIGHTS:
            raise ValueError(f"weights '{weights}' is not known (known: {', '.join(WEIGHTS)})")
        self.gated, self.renormalise = gate_proj is not None, weights == "chosen_softmax"
        if experts < 0 or identity < 0 or not (0 < top <= experts + identity):
            raise ValueError(f"{top} of {experts} + {identity} experts cannot be chosen")
        self.hidden, self.experts, self.identity, self.top = int(hidden), int(experts), int(identity), int(top)
        self.intermediate, self.activation = int(intermediate), activation
        self.names = dict(r=router, c=correction, u=up_proj, d=down_proj, g=gate_proj, b=router_bias)
        self.bias = None
        self.shared = build_part("feed_forward", shared) if shared is not None else None
        self.router = self.correction = self.up = self.down = None

    @property
    def outputs(self) -> int:
        return self.experts + self.identity

    def tensors(self):
        n = self.names
        t = {n["r"]: TensorSpec((self.outputs, self.hidden))}
        if n["c"] is not None:
            t[n["c"]] = TensorSpec((self.outputs,))
        if n["b"] is not None:
            t[n["b"]] = TensorSpec((self.outputs,))
        for e in range(self.experts):
            if self.gated:
                t[n["g"].format(e)] = TensorSpec((self.intermediate, self.hidden))
            t[n["u"].format(e)] = TensorSpec((self.intermediate, self.hidden))
            t[n["d"].format(e)] = TensorSpec((self.hidden, self.intermediate))
        if self.shared is not None:
            t.update(self.shared.tensors())
        return t

    def load(self, weights, device, dtype):
        n = self.names
        self.router = Linear(compute_form(weights[n["r"]], device, dtype), role="router")
        self.correction = weights[n["c"]].to(device).float().contiguous() if n["c"] is not None else None
        self.bias = weights[n["b"]].to(device).float().contiguous() if n["b"] is not None else None
        if self.experts:
            # every expert's matrix of a kind in one tensor [experts, out, in]: a grouped product picks its expert by index
            # (gated experts: an expert's gate rows, then its up rows)
            ups = [torch.cat([weights[n["g"].format(e)], weights[n["u"].format(e)]]) if self.gated else weights[n["u"].format(e)]
                   for e in range(self.experts)]
            self.up = compute_form(torch.stack(ups), device, dtype)
            self.down = compute_form(torch.stack([weights[n["d"].format(e)] for e in range(self.experts)]), device, dtype)
        if self.shared is not None:
            self.shared.load(weights, device, dtype)

    def first_weights(self):
        return self.router.weight if self.router is not None else None

    def _grouped_kernel(self, x: torch.Tensor, tokens: int) -> str:
        """Which grouped product runs the experts: few (token, choice) pairs meet mostly different experts, and the step costs
        what reading those experts' weights costs (the kernel for few rows); many pairs go to the tensor cores where the
        operands are bfloat16 with rows in whole 16-byte pieces; everything else to the general CUDA-core kernel."""
        same = self.up is not None and x.dtype == self.up.dtype
        pairs = tokens * self.top
        tensor_cores = same and x.dtype == torch.bfloat16 and self.hidden % 8 == 0 and self.intermediate % 8 == 0
        if same and pairs <= (SKINNY_PAIRS_BESIDE_TC if tensor_cores else SKINNY_MAX_PAIRS):
            return "skinny"
        return "tc" if tensor_cores else "simt"

    def _experts(self, x: torch.Tensor, ctx):
        """Routing, the sorted rows and the experts' products: (y, pair_row, weight), y float32 [sorted rows, hidden]."""
        T, dev = x.shape[0], x.device
        logits = self.router(x, out_dtype=torch.float32, ctx=ctx)
        chosen = torch.empty((T, self.top), dtype=torch.int32, device=dev)
        weight = torch.empty((T, self.top), dtype=torch.float32, device=dev)
        kernel = self._grouped_kernel(x, T)
        tile = ops.gemm_group_tile(kernel)
        tiles = ops.moe_tiles(T, self.top, self.experts, tile)
        ints = torch.empty(T * self.top + tiles * tile + tiles + 1 + max(self.experts, 1), dtype=torch.int32, device=dev)
        pair_row = ints[: T * self.top].view(T, self.top)
        row_token = ints[T * self.top: T * self.top + tiles * tile]
        tile_group = ints[T * self.top + tiles * tile: T * self.top + tiles * tile + tiles + 1]   # and the number of tiles in use
        counts = ints[T * self.top + tiles * tile + tiles + 1:]
        if T * self.top <= ops.MOE_SMALL_PAIRS and self.outputs <= 512:
            ops.moe_route_place(chosen, weight, pair_row, row_token, tile_group, logits, self.correction, self.experts, tile,
                                self.bias, self.renormalise)
        else:
            ops.moe_route(chosen, weight, logits, self.correction, self.bias, self.renormalise)
            ops.moe_place(pair_row, row_token, tile_group, counts, chosen, self.experts, tile)
        if not self.experts:
            return torch.empty((1, self.hidden), dtype=torch.float32, device=dev), pair_row, weight   # y is never read
        rows, gather = x, True
        if kernel == "tc":     # its tiles come by TMA, which reads rows side by side
            rows, gather = torch.empty((tiles * tile, self.hidden), dtype=x.dtype, device=dev), False
            ops.moe_gather(rows, x, row_token)
        ops.tag = "experts_up"
        if self.gated:
            both = torch.empty((tiles * tile, 2 * self.intermediate), dtype=x.dtype, device=dev)
            ops.gemm_grouped(kernel, both, rows, self.up, tile_group, row_token, gather, ops.EPILOGUE_STORE)
            act = torch.empty((tiles * tile, self.intermediate), dtype=x.dtype, device=dev)
            ops.gated_act(act, both, GATED_ACTIVATIONS[self.activation])   # (rows of tiles not in use hold whatever was there: nobody reads them)
        else:
            act = torch.empty((tiles * tile, self.intermediate), dtype=x.dtype, device=dev)
            ops.gemm_grouped(kernel, act, rows, self.up, tile_group, row_token, gather, ACTIVATIONS[self.activation])
        y = torch.empty((tiles * tile, self.hidden), dtype=torch.float32, device=dev)
        ops.tag = "experts_down"
        ops.gemm_grouped(kernel, y, act, self.down, tile_group, row_token, False, ops.EPILOGUE_STORE)
        ops.tag = None
        return y, pair_row, weight

    def forward(self, x: torch.Tensor, residual: torch.Tensor, ctx, store: bool = False) -> None:
        y, pair_row, weight = self._experts(x, ctx)
        ops.moe_combine(residual, y, x, pair_row, weight, add=not store)
        if self.shared is not None:
            self.shared.forward(x, residual, ctx)
        ctx.prenormed = None

    def forward_then_norm(self, x: torch.Tensor, residual: torch.Tensor, norm, ctx, rows_dtype=None):
        """residual += norm(mixture(x)) for a block whose norm stands behind the sublayer: the experts' rows are added up,
        normed and added to the residual by one kernel.  Returns the new residual rows rounded to `rows_dtype` (None: not
        wanted), or False when this part cannot do it for this norm (the block then goes the long way)."""
        if getattr(norm, "groups", 1) != 1 or self.hidden > ops.MOE_COMBINE_NORM_MAX_WIDTH or norm.dim != self.hidden:
            return False
        branch = None
        if self.shared is not None:
            branch = torch.empty_like(residual)
            if getattr(self.shared, "can_store", False):
                self.shared.forward(x, branch, ctx, store=True)
            else:
                branch.zero_()
                self.shared.forward(x, branch, ctx)
        y, pair_row, weight = self._experts(x, ctx)
        rows = torch.empty(residual.shape, dtype=rows_dtype, device=residual.device) if rows_dtype is not None else None
        ops.moe_combine_norm(residual, rows, branch, y, x, pair_row, weight, norm.gain, norm.eps)
        ctx.prenormed = None
        return rows


register_part("feed_forward", "routed_experts", RoutedExperts)
