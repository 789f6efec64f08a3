"""A weight matrix [out, in] and the choice of the matrix-product kernel for it."""
from __future__ import annotations

import torch

from ..kernels import fast, ops
from .base import Prenormed


def compute_form(t: torch.Tensor, device, dtype: torch.dtype) -> torch.Tensor:
    """A stored tensor as the engine computes with it: the 32-bit path widens everything
    to float32; the bfloat16 path keeps each tensor as it is stored (bfloat16, or 32-bit
    where the checkpoint has 32-bit)."""
    t = t.to(device)
    if dtype == torch.float32 and t.is_floating_point():
        t = t.to(torch.float32)
    return t.contiguous()


# Whether products that add into the residual prepare the norm that follows them (parts.base.Prenormed).  A switch, so that
# the two ways can be timed and compared against each other; both give the same result to bfloat16 rounding.
fold_norms = True


class Linear:
    """y = epilogue(x @ W^T) with W [out, in]; for the SwiGLU epilogue W is [2*out, in]."""

    def __init__(self, weight: torch.Tensor, epilogue: int = ops.EPILOGUE_STORE, role: str | None = None):
        self.weight = weight
        self.epilogue = epilogue
        self.role = role   # what a profile books this product under
        rows = weight.shape[0]
        self.out_features = rows // 2 if epilogue == ops.EPILOGUE_SWIGLU else rows
        self.in_features = weight.shape[1]

    def __call__(self, x, out: torch.Tensor | None = None, out_dtype: torch.dtype | None = None, ctx=None):
        """x: the activations, or a Prenormed (a norm's output in two pieces; `ctx` is then needed for the case that the
        kernel at hand cannot apply the row scale and the norm has to run after all)."""
        if out is None:
            out = torch.empty((x.shape[0], self.out_features), dtype=out_dtype or x.dtype, device=x.device)
        ops.tag = self.role
        try:
            if isinstance(x, Prenormed):
                if self.epilogue != ops.EPILOGUE_ACCUMULATE and fast.try_matmul(out, x.normed, self.weight, self.epilogue, x.row_scale()):
                    return out
                x = x.materialize(ctx)
            matmul(out, x, self.weight, self.epilogue)
        finally:
            ops.tag = None
        return out

    def add_then_norm(self, x: torch.Tensor, residual: torch.Tensor, norm, ctx) -> None:
        """residual += x @ W^T.  `norm` (or None) is the norm that will be applied to the residual rows next: where the
        kernel can, it also leaves that norm's input behind (ctx.prenormed), and the norm will not run."""
        if fold_norms and ctx is not None and norm is not None and getattr(norm, "foldable", False) and getattr(norm, "gain", None) is not None \
                and norm.dim == residual.shape[1] and residual.shape[0] == x.shape[0]:
            ops.tag = self.role
            try:
                left = fast.try_matmul_then_norm(residual, x, self.weight, norm.gain)
            finally:
                ops.tag = None
            if left is not None:
                ctx.prenormed = Prenormed(left[0], left[1], norm.dim, norm.eps, residual, norm)
                return
        if ctx is not None:
            ctx.prenormed = None
        self(x, out=residual)


TC_BATCH_MIN_TOKENS = 128   # from this many tokens on, a batch of small products goes to the tensor cores one by one,
TC_ALWAYS_MIN_WEIGHT = 512 * 512  # from this size of w[z] on, the tensor-core kernel at every number of tokens
TC_BATCH_MIN_WEIGHT = 256 * 256   # if each of them is large enough to be worth a launch of its own (entries of w[z])


def matmul_batched(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, x_step: int, out_step: int) -> None:
    """out[:, z*out_step : +N] = x[:, z*x_step : +K] @ w[z]^T for every z of w [batch, N, K]: the per-head or per-block
    products of a layer (a block-diagonal gate; a projection that every head has of its own).  Few tokens (a decode step):
    one CUDA-core launch for the whole batch, a warp per output column, which reads w once.  Many tokens: one tensor-core
    product per z where the kernel takes the operands.  Between the two: one CUDA-core launch in tiles."""
    batch, N, K = w.shape
    both_bf16 = x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16
    # products as large as a layer's own projections (time mixing's four) stream their weights best through the tensor-core
    # kernel at every number of tokens; a launch each costs less than the batched CUDA-core kernels lose on them
    large = both_bf16 and N * K >= TC_ALWAYS_MIN_WEIGHT
    if x.shape[0] <= ops.SKINNY_MAX_ROWS and x.dtype == w.dtype and not large:
        ops.gemm_skinny_batched(out, x, w, x_step, out_step)
        return
    if (x.shape[0] >= TC_BATCH_MIN_TOKENS or large) and N * K >= TC_BATCH_MIN_WEIGHT and both_bf16:
        views = [(out[:, z * out_step: z * out_step + N], x[:, z * x_step: z * x_step + K], w[z]) for z in range(batch)]
        if all(ops.gemm_tc_supported(o, a, b, ops.EPILOGUE_STORE) for o, a, b in views[:2]) and (x_step * 2) % 16 == 0:
            for o, a, b in views:
                ops.gemm_tc(o, a, b, ops.EPILOGUE_STORE, ops.device_status(o.device), checked=True)
            return
    if x.shape[0] <= ops.SKINNY_MAX_ROWS and x.dtype == w.dtype:
        ops.gemm_skinny_batched(out, x, w, x_step, out_step)
        return
    ops.gemm_simt_batched(out, x, w, batch, x_step, out_step)


def matmul(out: torch.Tensor, x: torch.Tensor, w: torch.Tensor, epilogue: int) -> None:
    """Picks the kernel: tensor-core kernels where they take the shape and types, else CUDA cores."""
    if fast.try_matmul(out, x, w, epilogue):
        return
    ops.gemm_simt(out, x, w, epilogue)
