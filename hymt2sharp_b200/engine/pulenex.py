"""Pulenex: from its configuration to a ModelSpec.

Every layer is a sandwich block whose norms are layer norms with a gain and no bias, before AND after each sublayer:
x += norm1b(mixer(norm1(x))), x += norm2b(ff(norm2(x))), the second line absent in a layer without a feed-forward.  The mixer
is retention with rotary positions on q and k; or latent attention in a sliding window with an output gate per head, whose
compressed rows a later layer may read instead of making its own (the order names the run whose cache plane it reads); or
two mixers side by side on the same input, chunked softmax attention whose heads talk and the gated delta rule, whose
outputs are each divided by their root mean square over the model width, multiplied by a stored gain, and averaged.  The
feed-forward is dense, gated, biased and clamped.  The final norm is a layer norm too, and the logits are scaled.  Tensor
names are those of the design's checkpoints: 'l<i>.' in front of a layer's, '.mix.' for its mixer, '.mlp.' for its
feed-forward.
"""
from __future__ import annotations

from ..config.pulenex import ARCHITECTURE, PulenexConfig
from ..config.registry import register_architecture
from ..parts.base import PartSpec
from .spec import ModelSpec, Run

GLU_ALPHA = 1.702        # the feed-forward's activation is g * sigmoid(1.702 g): a constant of the design
BRANCH_SCALE = 0.5       # a parallel layer's output is half the sum of its two normed branches


def build_spec(cfg: PulenexConfig) -> ModelSpec:
    W = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("layernorm", dict(dim=W, eps=cfg.norm_eps, weight=name))

    keep = cfg.cache_windows()
    layers, unread, order = [], [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        x = p + "mix."
        params = dict(norm1=norm(p + "norm1"), mixer=None, norm1_after=norm(p + "norm1b"))
        cache_from = None
        if layer.type == "retention":
            position = PartSpec("neox_rope", dict(head_dim=m.dim, rope_dim=m.rot.dims, base=m.rot.base)) if m.rot.dims else None
            params["mixer"] = PartSpec("retention", dict(hidden=W, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), eps=cfg.norm_eps,
                                                         q_proj=x + "q", k_proj=x + "k", v_proj=x + "v", g_proj=x + "g", o_proj=x + "o",
                                                         position=position))
        elif layer.type == "latent_attention":
            position = PartSpec("yarn_interleaved", dict(dims=m.rot.dims, base=m.rot.base, scaling=None)) if m.rot.dims else None
            cache_from = m.kv_from      # (layers run once each, so a layer's number is its place in the order)
            params["mixer"] = PartSpec("latent_attention", dict(
                hidden=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale, eps=cfg.norm_eps,
                position=position, gate="head", q_proj=x + "q", dkv_proj=x + "dkv", dkv_norm=x + "dkv.norm", uk_proj=x + "uk",
                uv_proj=x + "uv", o_proj=x + "o", g_proj=x + "g", window=m.window, own_kv=m.kv_from is None, cache_window=keep[i]))
        else:
            a, b = m.left, m.right
            l, r = x + "left.", x + "right."
            position = PartSpec("yarn_interleaved", dict(dims=a.rot.dims, base=a.rot.base, scaling=None)) if a.rot.dims else None
            left = PartSpec("talking_attention", dict(
                hidden=W, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, scale=a.scale, position=position, q_proj=l + "q", k_proj=l + "k",
                o_proj=l + "o", talk=l + "talk", temp=l + "temp", sink=l + "sink", g_proj=l + "g", mask="chunk" if a.chunk else None,
                mask_size=a.chunk or 0, taps=a.conv, q_conv=l + "q.conv", k_conv=l + "k.conv", values="keys"))
            right = PartSpec("gated_delta", dict(
                hidden=W, heads=b.heads, kv_heads=b.kv_heads, dim=b.dim, vdim=b.vdim, taps=b.conv, eps=cfg.norm_eps, q_proj=r + "q",
                k_proj=r + "k", v_proj=r + "v", q_conv=r + "q.conv", k_conv=r + "k.conv", v_conv=r + "v.conv", b_proj=r + "b",
                a_log=r + "A_log", a1_proj=r + "a1", a2_proj=r + "a2", dt_bias=r + "dt_bias", g1_proj=r + "g1", g2_proj=r + "g2",
                norm=r + "norm", o_proj=r + "o", decay_rank=b.decay_rank or -1, gate_rank=b.gate_rank or -1))
            params.update(mixers=[(left, l + "out", BRANCH_SCALE), (right, r + "out", BRANCH_SCALE)], mixers_eps=cfg.norm_eps)
        if layer.mlp is not None:
            f, y = layer.mlp, p + "mlp."
            params.update(norm2=norm(p + "norm2"), norm2_after=norm(p + "norm2b"),
                          feed_forward=PartSpec("clamped_glu", dict(hidden=W, intermediate=f.ff, limit=f.limit, alpha=GLU_ALPHA,
                                                                    gate_proj=y + "gate", up_proj=y + "up", down_proj=y + "down",
                                                                    gate_bias=y + "gate.b", up_bias=y + "up.b", down_bias=y + "down.b")))
        else:
            # a layer without a feed-forward reads none of the second sublayer's tensors, should a checkpoint hold them
            unread.append(rf"l{i}\.(norm2|norm2b|mlp\..*)")
        layers.append(PartSpec("sandwich", params))
        order.append(Run(i, cache_from=cache_from))
    return ModelSpec(vocab=cfg.vocab, hidden=W, embedding="embed", layers=layers, order=order, final_norm=norm("final.norm"),
                     head="head", logit_scale=cfg.logit_scale, ignorable_tensors=unread)


def tensor_shapes(cfg: PulenexConfig):
    from .model import DecoderModel
    return DecoderModel(build_spec(cfg)).tensors()


register_architecture(ARCHITECTURE, PulenexConfig, build_spec, tensor_shapes)
