"""RMSNorm part: y = x / sqrt(mean(x^2) + eps) * gain
(src/HyMT2Sharp/Ops.cs:29-89).  With `groups` > 1 a row is cut into that many equal
consecutive parts and each part is divided by its own root mean square; the gain
spans the whole row.  With `offset` the stored weight w lies around zero and the gain
is offset + w, added in float32 and kept so (a gain of 1 + w rounded to bfloat16 would
lose most of w)."""
from __future__ import annotations

import torch

from ..kernels import ops
from ..weights.loader import TensorSpec
from .base import register_part
from .linear import compute_form


class RMSNorm:
    graph_safe = True  # its forward only launches kernels on the current stream

    def __init__(self, dim: int, eps: float, weight: str, groups: int = 1, offset: float = 0.0):
        self.dim, self.eps, self.weight_name, self.groups = int(dim), float(eps), weight, int(groups)
        self.offset = float(offset)
        if self.groups < 1 or self.dim % self.groups:
            raise ValueError(f"a norm over {dim} entries cannot be cut into {groups} equal parts")
        # y = x * r * gain with ONE row scale r: the products around it can take it over (parts.base.Prenormed);
        # with several parts a row has several scales, and the norm runs as its own kernel
        self.foldable = self.groups == 1
        self.gain = None

    def tensors(self):
        return {self.weight_name: TensorSpec((self.dim,), init="normal" if self.offset else "gain")}

    def load(self, weights, device, dtype):
        if self.offset:
            self.gain = (weights[self.weight_name].to(device).float() + self.offset).contiguous()
        else:
            self.gain = compute_form(weights[self.weight_name], device, dtype)

    def forward(self, x: torch.Tensor, ctx, out_dtype: torch.dtype, rows_index: torch.Tensor | None = None,
                rows: int | None = None, scale: float = 1.0, fresh: bool = False):
        """The normed rows; or, when the product that last changed `x` prepared this very norm, what it left behind
        (a Prenormed, for a consumer that takes one).  `fresh`: compute in any case."""
        pre = getattr(ctx, "prenormed", None)
        if pre is not None and not fresh:
            ctx.prenormed = None
            if pre.norm is self and pre.source is x and rows_index is None and scale == 1.0 and pre.normed.dtype == out_dtype:
                return pre
        n = rows if rows is not None else (rows_index.shape[0] if rows_index is not None else x.shape[0])
        out = torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        if self.groups == 1:
            ops.rmsnorm(out, x, self.gain, self.eps, rows_index, scale)
        else:
            ops.rmsnorm_groups(out, x, self.gain, self.eps, self.groups, rows_index, scale)
        return out

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        """residual (float32) += norm(x): a sublayer's output that is normed before it joins the residual stream."""
        ops.rmsnorm_groups(residual, x, self.gain, self.eps, self.groups, add=True)

    def add_into_then(self, x: torch.Tensor, residual: torch.Tensor, following: "RMSNorm", out_dtype: torch.dtype) -> torch.Tensor:
        """add_into, and what `following` (the norm that reads the residual next) makes of the new rows: one kernel where
        the two norms cut their rows alike, two otherwise."""
        if (following.dim, following.groups) == (self.dim, self.groups) and following.gain.dtype == self.gain.dtype \
                and x.dtype == torch.float32 and x.shape == residual.shape:
            out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
            ops.rmsnorm_groups_add_norm(residual, x, self.gain, self.eps, out, following.gain, following.eps, self.groups)
            return out
        self.add_into(x, residual)
        return following.forward(residual, None, out_dtype, fresh=True)


    def add_into_then_rows(self, x: torch.Tensor, residual: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        """add_into, and the new rows in `out_dtype` for a sublayer that reads the residual as it is (no norm in front of it):
        the residual itself where that is its type, else its rounding, written by the same kernel."""
        if out_dtype == residual.dtype:
            self.add_into(x, residual)
            return residual
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        ops.rmsnorm_add_then_rows(residual, x, self.gain, self.eps, out, self.groups)
        return out


register_part("norm", "rmsnorm", RMSNorm)


class LayerNorm:
    """Layer norm with a gain and no bias: y = (x - mean) / sqrt(variance + eps) * gain, the variance being the mean of the squared
    deviations; all in float32.  It offers what RMSNorm offers to a block with norms before and after its sublayers (forward,
    add_into, add_into_then, add_into_then_rows).  It cannot be folded into the products around it: a row has a mean to take
    off besides its scale."""
    graph_safe = True
    foldable = False

    def __init__(self, dim: int, eps: float, weight: str):
        self.dim, self.eps, self.weight_name = int(dim), float(eps), weight
        self.gain = None

    def tensors(self):
        return {self.weight_name: TensorSpec((self.dim,), init="gain")}

    def load(self, weights, device, dtype):
        self.gain = compute_form(weights[self.weight_name], device, dtype)

    def forward(self, x: torch.Tensor, ctx, out_dtype: torch.dtype, rows_index: torch.Tensor | None = None,
                rows: int | None = None, scale: float = 1.0, fresh: bool = False):
        if ctx is not None and getattr(ctx, "prenormed", None) is not None:
            ctx.prenormed = None     # (left for another norm; this one always runs)
        n = rows if rows is not None else (rows_index.shape[0] if rows_index is not None else x.shape[0])
        out = torch.empty((n, self.dim), dtype=out_dtype, device=x.device)
        ops.layernorm(out, x, self.gain, self.eps, rows_index, scale)
        return out

    def add_into(self, x: torch.Tensor, residual: torch.Tensor) -> None:
        """residual (float32) += norm(x)."""
        ops.layernorm(residual, x, self.gain, self.eps, add=True)

    def add_into_then(self, x: torch.Tensor, residual: torch.Tensor, following, out_dtype: torch.dtype) -> torch.Tensor:
        """add_into, and what `following` (the norm that reads the residual next) makes of the new rows: one kernel where that
        is a layer norm of the same width too, two otherwise."""
        if isinstance(following, LayerNorm) and following.dim == self.dim and following.gain.dtype == self.gain.dtype \
                and x.dtype == torch.float32 and x.shape == residual.shape:
            out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
            ops.layernorm_add_norm(residual, x, self.gain, self.eps, out, following.gain, following.eps)
            return out
        self.add_into(x, residual)
        return following.forward(residual, None, out_dtype, fresh=True)

    def add_into_then_rows(self, x: torch.Tensor, residual: torch.Tensor, out_dtype: torch.dtype) -> torch.Tensor:
        if out_dtype == residual.dtype:
            self.add_into(x, residual)
            return residual
        out = torch.empty(residual.shape, dtype=out_dtype, device=residual.device)
        ops.layernorm_add_norm(residual, x, self.gain, self.eps, out, None, 0.0)
        return out


register_part("norm", "layernorm", LayerNorm)
