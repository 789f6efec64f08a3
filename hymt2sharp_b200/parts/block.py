"""Pre-norm residual block: h += mixer(norm1(h)); h += ffn(norm2(h))
(src/HyMT2Sharp/HunyuanDenseModel.Prefill.cs:14-36).  The residual stream h is
float32; the normed activations have the engine's compute type."""
from __future__ import annotations

from ..kernels import ops
from .base import PartSpec, Prenormed, build_part, register_part


class PreNormBlock:
    def __init__(self, norm1: PartSpec, mixer: PartSpec, norm2: PartSpec, feed_forward: PartSpec):
        self.norm1 = build_part("norm", norm1)
        self.mixer = build_part("mixer", mixer)
        self.norm2 = build_part("norm", norm2)
        self.feed_forward = build_part("feed_forward", feed_forward)

    def parts(self):
        return (self.norm1, self.mixer, self.norm2, self.feed_forward)

    # -- what the model asks a block (never its parts): one entry per mixer it holds ---------------
    def cache_needs(self) -> list:
        return [self.mixer.cache_need()]

    def state_bytes(self) -> list:
        return [int(self.mixer.state_bytes())]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        t = {}
        for p in self.parts():
            t.update(p.tensors())
        return t

    def load(self, weights, device, dtype):
        for p in self.parts():
            p.load(weights, device, dtype)

    def first_norm(self):
        """The norm that this block applies to the residual first, if the part behind it can take a norm's output in
        two pieces (parts.base.Prenormed): the block before may then prepare it in its last product."""
        return self.norm1 if getattr(self.mixer, "takes_prenormed", False) else None

    def forward(self, residual, ctx, slots) -> None:
        x = self.norm1.forward(residual, ctx, ctx.dtype)      # what the block before left behind, or the norm's own kernel
        if isinstance(x, Prenormed) and not getattr(self.mixer, "takes_prenormed", False):
            x = x.materialize(ctx)
        # what the feed-forward streams first, for a mixer whose last kernel can ask for it ahead of time
        ctx.weights_ahead = getattr(self.feed_forward, "first_weights", lambda: None)()
        # the norm that comes next, for a mixer whose last product can prepare it
        ctx.norm_ahead = self.norm2 if getattr(self.feed_forward, "takes_prenormed", False) else None
        self.mixer.forward(x, residual, ctx, slots[0])
        ctx.weights_ahead = ctx.norm_ahead = None
        x = self.norm2.forward(residual, ctx, ctx.dtype)
        if isinstance(x, Prenormed) and not getattr(self.feed_forward, "takes_prenormed", False):
            x = x.materialize(ctx)
        ctx.norm_ahead = ctx.next_first_norm
        self.feed_forward.forward(x, residual, ctx)
        ctx.norm_ahead = None


register_part("block", "pre_norm", PreNormBlock)


class SandwichBlock:
    """A block with a norm before AND after each sublayer, and an optional short convolution in front of each:

        h = norm1(x);  h = h + conv1(h);  x += norm1b(mixer(h))
        h = norm2(x);  h = h + conv2(h);  x += norm2b(ff(h))          (no feed-forward: the second line is absent)

    The convolutions run over time on each channel (parts.conv.ShortConv); their last inputs are state of the
    sequence, which this block asks the model for beside its mixer's: cache_needs() / state_bytes() have the mixer's
    entry first, then one entry for each convolution it holds.  A sublayer's output is collected in a float32 buffer and
    joins the residual through the norm after it.  Mixers and feed-forwards add into what they are given, so the buffer
    starts from zeros; a part that says `can_store = True` takes `store=True` and overwrites it instead (no zeroing).

    The norms in FRONT are optional (`norm1` / `norm2` None): such a sublayer reads the residual rows themselves, and the norm
    is on its output only, x += norm1b(mixer(x)).  In an engine whose compute type is not float32 the rows are rounded once;
    the kernel of the norm behind a sublayer writes that rounding beside the new residual, also for the block that runs next
    (left in `ctx.shared["residual_rows"]`).

    Several mixers side by side (`mixers` = [(PartSpec, gain tensor name, scale), ...] in place of `mixer`): all read the same h,
    each has its own cache plane and state (cache_needs() / state_bytes() list them first, in order), and the first sublayer's
    output is sum_i scale_i * y_i / sqrt(mean(y_i^2) + mixers_eps) * gain_i: every mixer's output is divided by its own root
    mean square over the model width and multiplied by its own stored gain before the sum (one kernel)."""

    def __init__(self, norm1: PartSpec | None, mixer: PartSpec | None, norm1_after: PartSpec, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, norm2_after: PartSpec | None = None, conv1: dict | None = None,
                 conv2: dict | None = None, mixers: list | None = None, mixers_eps: float = 0.0):
        from .conv import ShortConv
        if (mixer is None) == (not mixers):
            raise ValueError("a block holds one mixer (`mixer`) or several side by side (`mixers`), not both and not neither")
        if mixers and len(mixers) > ops.MAX_NORMED_BRANCHES:
            raise ValueError(f"{len(mixers)} mixers side by side (at most {ops.MAX_NORMED_BRANCHES})")
        self.norm1 = build_part("norm", norm1) if norm1 is not None else None
        self.side = [build_part("mixer", m) for m, _, _ in mixers] if mixers else []
        self.side_names = [name for _, name, _ in mixers] if mixers else []
        self.side_scales = [float(sc) for _, _, sc in mixers] if mixers else []
        self.side_eps, self.side_gains = float(mixers_eps), []
        self.mixer = build_part("mixer", mixer) if mixer is not None else None
        self.norm1_after = build_part("norm", norm1_after)
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.norm2 = build_part("norm", norm2) if feed_forward is not None and norm2 is not None else None
        self.norm2_after = build_part("norm", norm2_after) if feed_forward is not None else None
        self.conv1 = ShortConv(add_input=True, **conv1) if conv1 is not None else None
        self.conv2 = ShortConv(add_input=True, **conv2) if conv2 is not None and feed_forward is not None else None

    def parts(self):
        return tuple(p for p in (self.norm1, self.conv1, self.mixer, *self.side, self.norm1_after, self.norm2, self.conv2,
                                 self.feed_forward, self.norm2_after) if p is not None)

    def _convs(self):
        return [c for c in (self.conv1, self.conv2) if c is not None]

    def _mixers(self):
        return [self.mixer] if self.mixer is not None else self.side

    def cache_needs(self) -> list:
        return [m.cache_need() for m in self._mixers()] + [None for _ in self._convs()]

    def state_bytes(self) -> list:
        return [int(m.state_bytes()) for m in self._mixers()] + [c.state_bytes() for c in self._convs()]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        from ..weights.loader import TensorSpec
        t = {}
        for p in self.parts():
            t.update(p.tensors())
        width = self.norm1_after.dim
        for name in self.side_names:
            t[name] = TensorSpec((width,), init="gain")
        return t

    def load(self, weights, device, dtype):
        from .linear import compute_form
        for p in self.parts():
            p.load(weights, device, dtype)
        self.side_gains = [compute_form(weights[name], device, dtype) for name in self.side_names]

    def first_norm(self):
        return None   # what reads the residual first here is followed by a convolution, which wants the plain rows

    def forward(self, residual, ctx, slots) -> None:
        import torch
        conv_slots = list(slots[len(self._mixers()):])
        ctx.weights_ahead = ctx.norm_ahead = None
        left = ctx.shared.pop("residual_rows", None)
        if self.norm1 is not None:
            h = self.norm1.forward(residual, ctx, ctx.dtype, fresh=True)
        elif left is not None and left[0] is residual and left[1].dtype == ctx.dtype:
            h = left[1]                      # what the block in front wrote beside its last change of the residual
        else:
            h = self._rows(residual, ctx)
        if self.conv1 is not None:
            h = self.conv1.forward(h, ctx, conv_slots.pop(0))
        if self.side:
            outs = []
            for mixer, slot in zip(self.side, slots):
                y = torch.empty_like(residual) if getattr(mixer, "can_store", False) else torch.zeros_like(residual)
                mixer.forward(h, y, ctx, slot, **({"store": True} if getattr(mixer, "can_store", False) else {}))
                outs.append(y)
            branch = torch.empty_like(residual)
            ops.rmsnorm_sum(branch, outs, self.side_gains, self.side_scales, self.side_eps)
        elif getattr(self.mixer, "can_store", False):
            branch = torch.empty_like(residual)
            self.mixer.forward(h, branch, ctx, slots[0], store=True)
        else:
            branch = torch.zeros_like(residual)
            self.mixer.forward(h, branch, ctx, slots[0])
        ctx.prenormed = None
        if self.feed_forward is None:
            self._last(self.norm1_after, branch, residual, ctx)
            return
        if self.norm2 is not None:
            h = self.norm1_after.add_into_then(branch, residual, self.norm2, ctx.dtype)
        else:
            h = self.norm1_after.add_into_then_rows(branch, residual, ctx.dtype)
        if self.conv2 is not None:
            h = self.conv2.forward(h, ctx, conv_slots.pop(0))
        if hasattr(self.feed_forward, "forward_then_norm"):
            # a feed-forward that adds its own pieces up can norm them and add them to the residual on the way
            want = ctx.dtype if self.norm1 is None and ctx.dtype != residual.dtype else None
            rows = self.feed_forward.forward_then_norm(h, residual, self.norm2_after, ctx, want)
            if rows is not False:
                if rows is not None:
                    ctx.shared["residual_rows"] = (residual, rows)
                return
        if getattr(self.feed_forward, "can_store", False):
            self.feed_forward.forward(h, branch, ctx, store=True)
        else:
            branch.zero_()
            self.feed_forward.forward(h, branch, ctx)
        ctx.prenormed = None
        self._last(self.norm2_after, branch, residual, ctx)

    @staticmethod
    def _rows(residual, ctx):
        """The residual rows as a sublayer without a norm in front reads them: themselves, or rounded to the compute type."""
        import torch
        if ctx.dtype == residual.dtype:
            return residual
        h = torch.empty(residual.shape, dtype=ctx.dtype, device=residual.device)
        ops.convert(h, residual)
        return h

    def _last(self, norm, branch, residual, ctx) -> None:
        """The block's last change of the residual.  A block whose own first sublayer reads plain rows expects the same of the
        block behind it and leaves the rounded rows for it."""
        if self.norm1 is None and ctx.dtype != residual.dtype:
            ctx.shared["residual_rows"] = (residual, norm.add_into_then_rows(branch, residual, ctx.dtype))
        else:
            norm.add_into(branch, residual)


register_part("block", "sandwich", SandwichBlock)


class StreamsBlock:
    """A pre-norm block over a residual that is kept as several streams (hyper-connections), with any number of mixers side
    by side.  X is float32 [streams, T, hidden]; for sublayer q (1: the mixers, 2: the feed-forward) with the stored vectors
    in_q, out_q [streams] and the matrix mix_q [streams, streams], indexed [from, to]:

        u = sum_s in_q[s] X[s];   y = sublayer(norm_q(u));   X[r] <- sum_s mix_q[s, r] X[s] + out_q[r] * y   (every r from the old X)

    The first sublayer's y is sum_i scale_i * mixer_i(norm_1(u)): the mixers read the same rows, each has its own cache
    plane or state (cache_needs() / state_bytes() list them in order) and writes a float32 buffer of its own; the scales
    are applied in float32 where the buffers are added.  `hyper1` / `hyper2` None: one stream without stored tables, which is
    the plain residual sum X <- X + y.  The write of a sublayer and the read and norm of the next one (this block's
    feed-forward, or the first sublayer of the block that runs next, `ctx.block_ahead`) are one kernel; the rows that such
    a kernel prepared wait in `ctx.shared["stream_rows"]`."""

    def __init__(self, streams: int, norm1: PartSpec, mixers: list, norm2: PartSpec | None = None,
                 feed_forward: PartSpec | None = None, hyper1: dict | None = None, hyper2: dict | None = None):
        """`mixers`: [(PartSpec, scale), ...]; `hyper1` / `hyper2`: {"in": name, "out": name, "mix": name} of the stored tables."""
        if not mixers or len(mixers) > ops.MAX_BRANCHES:
            raise ValueError(f"a block holds 1 to {ops.MAX_BRANCHES} mixers side by side, got {len(mixers)}")
        if not (1 <= streams <= ops.MAX_STREAMS):
            raise ValueError(f"{streams} streams (1 to {ops.MAX_STREAMS})")
        if (hyper1 is None or (feed_forward is not None and hyper2 is None)) and streams != 1:
            raise ValueError("several streams need the tables that mix them")
        self.streams = int(streams)
        self.norm1 = build_part("norm", norm1)
        self.mixers = [build_part("mixer", m) for m, _ in mixers]
        self.scales = [float(s) for _, s in mixers]
        self.feed_forward = build_part("feed_forward", feed_forward) if feed_forward is not None else None
        self.norm2 = build_part("norm", norm2) if feed_forward is not None else None
        self.names = [hyper1, hyper2 if feed_forward is not None else None]
        self.tables = [None, None]     # per sublayer: (w_in, w_out, mix) float32 on the device

    def parts(self):
        return tuple(p for p in (self.norm1, *self.mixers, self.norm2, self.feed_forward) if p is not None)

    def cache_needs(self) -> list:
        return [m.cache_need() for m in self.mixers]

    def state_bytes(self) -> list:
        return [int(m.state_bytes()) for m in self.mixers]

    @property
    def graph_safe(self) -> bool:
        return all(getattr(p, "graph_safe", False) for p in self.parts())

    def tensors(self):
        from ..weights.loader import TensorSpec
        t, S = {}, self.streams
        for p in self.parts():
            t.update(p.tensors())
        for names in self.names:
            if names is not None:
                t[names["in"]] = TensorSpec((S,), init="gain")
                t[names["out"]] = TensorSpec((S,), init="gain")
                t[names["mix"]] = TensorSpec((S, S), init="identity")
        return t

    def load(self, weights, device, dtype):
        import torch
        for p in self.parts():
            p.load(weights, device, dtype)
        for q, names in enumerate(self.names):
            if names is not None:
                self.tables[q] = tuple(weights[names[k]].to(device).float().reshape(-1).contiguous() for k in ("in", "out", "mix"))
            else:
                self.tables[q] = tuple(torch.ones(1, dtype=torch.float32, device=device) for _ in range(3))

    def first_norm(self):
        return None   # (the products of the block in front cannot prepare this block's input: it is a mixture of streams)

    def first_read(self):
        """What the block in front needs to prepare this block's first input: (w_in, norm)."""
        return self.tables[0][0], self.norm1

    def _read(self, X, w_in, norm, ctx):
        import torch
        out = torch.empty(X.shape[1:], dtype=ctx.dtype, device=X.device)
        return ops.streams_step(X, read=(w_in, norm.gain, norm.eps, out))

    def _write(self, X, q: int, branches, scales, ctx, ahead):
        """Sublayer q's outputs go into the streams; `ahead` = (w_in, norm) of the read that follows (or None)."""
        import torch
        _, w_out, mix = self.tables[q]
        if ahead is None:
            ops.streams_step(X, write=(mix, w_out, branches, scales))
            return None
        w_in, norm = ahead
        out = torch.empty(X.shape[1:], dtype=ctx.dtype, device=X.device)
        return ops.streams_step(X, write=(mix, w_out, branches, scales), read=(w_in, norm.gain, norm.eps, out))

    def forward(self, residual, ctx, slots) -> None:
        import torch
        X = residual
        if X.dim() != 3 or X.shape[0] != self.streams:
            raise ValueError(f"this block reads {self.streams} residual streams [streams, T, hidden], got {tuple(X.shape)}")
        ctx.weights_ahead = ctx.norm_ahead = ctx.prenormed = None
        left = ctx.shared.pop("stream_rows", None)
        if left is not None and left[0] is X and left[1] is self:
            h = left[2]
        else:
            h = self._read(X, self.tables[0][0], self.norm1, ctx)
        branches = []
        for mixer, slot in zip(self.mixers, slots):
            y = torch.empty(X.shape[1:], dtype=torch.float32, device=X.device)
            mixer.forward(h, y, ctx, slot, store=True)
            branches.append(y)
        ctx.prenormed = None
        nxt = getattr(ctx, "block_ahead", None)
        after = nxt.first_read() if nxt is not None and hasattr(nxt, "first_read") and getattr(nxt, "streams", None) == self.streams else None
        if self.feed_forward is None:
            rows = self._write(X, 0, branches, self.scales, ctx, after)
        else:
            h = self._write(X, 0, branches, self.scales, ctx, (self.tables[1][0], self.norm2))
            y = branches[0]
            self.feed_forward.forward(h, y, ctx, store=True)
            ctx.prenormed = None
            rows = self._write(X, 1, [y], [1.0], ctx, after)
        if rows is not None:
            ctx.shared["stream_rows"] = (X, nxt, rows)


register_part("block", "streams", StreamsBlock)
