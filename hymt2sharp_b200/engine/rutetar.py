"""Rutetar: from its configuration to a ModelSpec.

Every layer is a pre-norm block over a residual kept as several streams (parts.block.StreamsBlock), whose norms store
their weight around zero (gain 1 + w).  The mixer is retention (linear attention with a fixed decay per head), or two
mixers side by side that read the same rows and are added with two scales: softmax attention in a sliding window with
biases, a partial rotation and an output gate per head, and time mixing with a decay per token and channel.  The
feed-forward is dense and gated with the tanh form of GELU, a mixture of SiLU-gated experts whose router has a bias and
whose weights are the softmax over the chosen outputs alone, or absent.  A stretch of layers runs several times in a row
with the same weights, every run with its own cache plane and state (the order names the layer again).  Tensor names are
those of the design's checkpoints: 'l<i>.' in front of a layer's, '.mix.' for its mixer, '.mlp.' for its feed-forward,
'.hc1.' / '.hc2.' for the tables of the streams.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.rutetar import ARCHITECTURE, RutetarConfig
from ..parts.base import PartSpec
from .spec import ModelSpec, Run

NORM_OFFSET = 1.0                 # a norm's gain is 1 + its stored weight
DENSE_ACTIVATION = "gelu_tanh"    # constants of the design
EXPERT_ACTIVATION = "silu"


def build_spec(cfg: RutetarConfig) -> ModelSpec:
    H = cfg.width

    def norm(name: str) -> PartSpec:
        return PartSpec("rmsnorm", dict(dim=H, eps=cfg.norm_eps, weight=name, offset=NORM_OFFSET))

    def tables(p: str, q: int):
        return None if cfg.streams is None else {k: f"{p}hc{q}.{k}" for k in ("in", "out", "mix")}

    layers, unread = [], []
    for i, layer in enumerate(cfg.layers):
        p, m = f"l{i}.", layer.mixer
        x = p + "mix."
        if layer.type == "retention":
            mixers = [(PartSpec("retention", dict(hidden=H, heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), eps=cfg.norm_eps,
                                                  q_proj=x + "q", k_proj=x + "k", v_proj=x + "v", g_proj=x + "g", o_proj=x + "o")), 1.0)]
        else:
            a, b = m.left, m.right
            l, r = x + "left.", x + "right."
            position = PartSpec("wavelength_scaled_rope", dict(dims=a.rot_dims, base=a.rot_base, scaling=None))
            left = PartSpec("gqa_attention", dict(
                hidden=H, heads=a.heads, kv_heads=a.kv_heads, head_dim=a.dim, value_dim=a.vdim, scale=a.scale, eps=cfg.norm_eps,
                qk_norm=False, window=a.window, position=position, q_proj=l + "q", k_proj=l + "k", v_proj=l + "v", o_proj=l + "o",
                q_bias=l + "q.b", k_bias=l + "k.b", v_bias=l + "v.b", head_gate=l + "g"))
            right = PartSpec("time_mix", dict(
                hidden=H, heads=b.heads, dim=b.dim, eps=cfg.norm_eps, decay_rank=b.rank, mu=r + "mu.{}", r_proj=r + "r", k_proj=r + "k",
                v_proj=r + "v", g_proj=r + "g", w1_proj=r + "w1", w2_proj=r + "w2", w0=r + "w0", bonus=r + "u", norm=r + "norm",
                o_proj=r + "o"))
            mixers = [(left, m.left_scale), (right, m.right_scale)]
        params = dict(streams=cfg.streams or 1, norm1=norm(p + "norm1"), mixers=mixers, hyper1=tables(p, 1))
        if layer.mlp is not None:
            f, y = layer.mlp, p + "mlp."
            if f.kind == "dense":
                ff = PartSpec("swiglu", dict(hidden=H, intermediate=f.ff, activation=DENSE_ACTIVATION, gate_proj=y + "gate",
                                             up_proj=y + "up", down_proj=y + "down"))
            else:
                ff = PartSpec("routed_experts", dict(
                    hidden=H, experts=f.experts, identity=0, top=f.top, intermediate=f.ff, activation=EXPERT_ACTIVATION,
                    router=y + "router", router_bias=y + "router.b", weights="chosen_softmax", gate_proj=y + "e{}.gate",
                    up_proj=y + "e{}.up", down_proj=y + "e{}.down"))
            params.update(norm2=norm(p + "norm2"), feed_forward=ff, hyper2=tables(p, 2))
        else:
            # a layer without a feed-forward reads none of the second sublayer's tensors, should a checkpoint hold them
            unread.append(rf"l{i}\.(norm2|hc2\..*|mlp\..*)")
        layers.append(PartSpec("streams", params))
    return ModelSpec(vocab=cfg.vocab, hidden=H, embedding="embed", layers=layers, order=[Run(i) for i in cfg.order()],
                     final_norm=norm("final.norm"), head="head", ignorable_tensors=unread, residual_streams=cfg.streams or 1)


def tensor_shapes(cfg: RutetarConfig):
    from .model import DecoderModel
    return DecoderModel(build_spec(cfg)).tensors()


register_architecture(ARCHITECTURE, RutetarConfig, build_spec, tensor_shapes)
