"""Configuration of the Pulenex design (config.json "architecture": "Pulenex").

A decoder whose layers are listed one by one: each entry of `layers` names its mixer (`type`), the mixer's sizes (`mixer`)
and its feed-forward (`mlp`, or null).  Mixer 'retention' is linear attention with a fixed decay per head and rotary
positions; mixer 'parallel' runs two mixers side by side on the same input, softmax attention in chunks whose heads talk
(`left`) and the gated delta rule (`right`), and averages their normed outputs; mixer 'latent_attention' is attention over a
compressed key/value row in a sliding window, which a later layer may read instead of making its own (`kv_from`).  The
feed-forward is dense and gated with clamps.  Every size and every constant that can differ between two models of the
design is read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ConfigReader

ARCHITECTURE = "Pulenex"
MIXERS = ("retention", "parallel", "latent_attention")
MLP_KINDS = ("dense",)


@dataclass(frozen=True)
class RotConfig:
    dims: int                # rotated entries of every head (the first ones), even; 0: none
    base: float


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple             # one constant per head
    rot: RotConfig


@dataclass(frozen=True)
class TalkingAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int                # the values are the keys, so it equals dim
    scale: float
    conv: int                # taps of the convolution on q and k
    chunk: int | None        # positions of a chunk; None: every token sees all before it
    rot: RotConfig


@dataclass(frozen=True)
class GatedDeltaConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int
    decay_rank: int | None   # widths of the decay's and the gate's inner projections; None: whatever the checkpoint's tensors hold
    gate_rank: int | None


@dataclass(frozen=True)
class ParallelConfig:
    left: TalkingAttentionConfig
    right: GatedDeltaConfig


@dataclass(frozen=True)
class LatentAttentionConfig:
    heads: int
    dim: int                 # per head: unrotated query/key entries
    rot_dim: int             # per head: rotated query entries; the one rotated key part that all heads share
    vdim: int
    kv_rank: int
    scale: float
    window: int | None       # positions that a token sees, itself included; None: all before it
    rot: RotConfig
    kv_from: int | None      # the layer whose compressed rows this one reads; None: its own


@dataclass(frozen=True)
class MlpConfig:
    kind: str
    ff: int
    limit: float


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object
    mlp: MlpConfig | None


def _rot(e: ConfigReader, prefix: str, dim: int, where: str) -> RotConfig:
    rot = RotConfig(dims=e.integer(prefix + "rot.dims", default=0, minimum=0),
                    base=e.number(prefix + "rot.base", default=10000.0, exclusive_minimum=0.0))
    if rot.dims % 2 or rot.dims > dim:
        raise ConfigError(f"{where}: {prefix}rot.dims {rot.dims} must be even and at most {dim}")
    return rot


@dataclass(frozen=True)
class PulenexConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    logit_scale: float | None
    raw: dict = field(compare=False, repr=False, default_factory=dict)

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, data: dict, source: str = "config.json") -> "PulenexConfig":
        r = ConfigReader(data, source)
        width = r.integer("width", minimum=1)
        entries = data.get("layers")
        if not isinstance(entries, list) or not entries:
            raise ConfigError(f"{source}: key 'layers' must be a list with at least one layer")
        layers = []
        for i, entry in enumerate(entries):
            where = f"{source}: layers[{i}]"
            if not isinstance(entry, dict):
                raise ConfigError(f"{where} must be an object")
            e = ConfigReader(entry, where)
            kind = e.string("type")
            if kind not in MIXERS:
                raise ConfigError(f"{where}: type '{kind}' is not known (known: {', '.join(MIXERS)})")
            if kind == "retention":
                heads, dim = e.integer("mixer.heads", minimum=1), e.integer("mixer.dim", minimum=1)
                decay = entry["mixer"].get("decay")
                if not isinstance(decay, list) or len(decay) != heads or \
                        not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                    raise ConfigError(f"{where}: mixer.decay must be a list of {heads} numbers, one per head")
                mixer = RetentionConfig(heads=heads, dim=dim, vdim=e.integer("mixer.vdim", minimum=1),
                                        decay=tuple(float(d) for d in decay), rot=_rot(e, "mixer.", dim, where))
            elif kind == "parallel":
                dim = e.integer("mixer.left.dim", minimum=1)
                left = TalkingAttentionConfig(
                    heads=e.integer("mixer.left.heads", minimum=1), kv_heads=e.integer("mixer.left.kv_heads", minimum=1), dim=dim,
                    vdim=e.integer("mixer.left.vdim", default=dim, minimum=1), scale=e.number("mixer.left.scale", exclusive_minimum=0.0),
                    conv=e.integer("mixer.left.conv", minimum=1), chunk=e.integer("mixer.left.mask.size", default=None, minimum=1),
                    rot=_rot(e, "mixer.left.", dim, where))
                if left.heads % left.kv_heads:
                    raise ConfigError(f"{where}: mixer.left.heads {left.heads} is not a multiple of mixer.left.kv_heads {left.kv_heads}")
                if left.vdim != dim:
                    raise ConfigError(f"{where}: mixer.left.vdim {left.vdim} differs from mixer.left.dim {dim}, but the values are the keys")
                right = GatedDeltaConfig(
                    heads=e.integer("mixer.right.heads", minimum=1), kv_heads=e.integer("mixer.right.kv_heads", minimum=1),
                    dim=e.integer("mixer.right.dim", minimum=1), vdim=e.integer("mixer.right.vdim", minimum=1),
                    conv=e.integer("mixer.right.conv", minimum=1), decay_rank=e.integer("mixer.right.decay_rank", default=None, minimum=1),
                    gate_rank=e.integer("mixer.right.gate_rank", default=None, minimum=1))
                if right.heads % right.kv_heads:
                    raise ConfigError(f"{where}: mixer.right.heads {right.heads} is not a multiple of mixer.right.kv_heads {right.kv_heads}")
                mixer = ParallelConfig(left=left, right=right)
            else:
                rot_dim = e.integer("mixer.rot_dim", minimum=0)
                mixer = LatentAttentionConfig(
                    heads=e.integer("mixer.heads", minimum=1), dim=e.integer("mixer.dim", minimum=0), rot_dim=rot_dim,
                    vdim=e.integer("mixer.vdim", minimum=1), kv_rank=e.integer("mixer.kv_rank", minimum=1),
                    scale=e.number("mixer.scale", exclusive_minimum=0.0), window=e.integer("mixer.mask.size", default=None, minimum=1),
                    rot=RotConfig(dims=e.integer("mixer.rot.dims", default=rot_dim, minimum=0),
                                  base=e.number("mixer.rot.base", default=10000.0, exclusive_minimum=0.0)),
                    kv_from=e.integer("mixer.kv_from", default=None, minimum=0))
                if mixer.rot.dims % 2 or mixer.rot.dims > rot_dim:
                    raise ConfigError(f"{where}: mixer.rot.dims {mixer.rot.dims} must be even and at most mixer.rot_dim {rot_dim}")
                if mixer.kv_from is not None:
                    j = mixer.kv_from
                    src = layers[j].mixer if j < i and layers[j].type == "latent_attention" else None
                    if src is None or src.kv_from is not None:
                        raise ConfigError(f"{where}: mixer.kv_from {j} must name an earlier latent_attention layer with rows of its own")
                    if (src.kv_rank, src.rot_dim, src.rot) != (mixer.kv_rank, mixer.rot_dim, mixer.rot):
                        raise ConfigError(f"{where}: mixer.kv_from {j}: that layer's kv_rank, rot_dim and rot differ from this layer's")
            mlp = None
            if entry.get("mlp") is not None:
                mlp_kind = e.string("mlp.kind")
                if mlp_kind not in MLP_KINDS:
                    raise ConfigError(f"{where}: mlp.kind '{mlp_kind}' is not known (known: {', '.join(MLP_KINDS)})")
                mlp = MlpConfig("dense", ff=e.integer("mlp.ff", minimum=1), limit=e.number("mlp.limit", exclusive_minimum=0.0))
            layers.append(LayerConfig(kind, mixer, mlp))
        return cls(vocab=r.integer("vocab", minimum=1), width=width, layers=tuple(layers),
                   norm_eps=r.number("norm.eps", exclusive_minimum=0.0), logit_scale=r.number("logit_scale", default=None), raw=data)

    def cache_windows(self) -> dict:
        """For every latent_attention layer: the positions that the cache has to keep of the rows it reads, which is the
        widest window among the layers that read the same rows (0: everything, as soon as one of them has no window)."""
        widest: dict = {}
        for i, l in enumerate(self.layers):
            if l.type == "latent_attention":
                src = i if l.mixer.kv_from is None else l.mixer.kv_from
                w = l.mixer.window or 0
                widest[src] = w if src not in widest else (0 if 0 in (w, widest[src]) else max(w, widest[src]))
        return {i: widest[i if l.mixer.kv_from is None else l.mixer.kv_from]
                for i, l in enumerate(self.layers) if l.type == "latent_attention"}

    # (what the command line prints about a loaded model)
    @property
    def num_hidden_layers(self) -> int:
        return len(self.layers)

    @property
    def hidden_size(self) -> int:
        return self.width

    @property
    def vocab_size(self) -> int:
        return self.vocab

    def to_dict(self) -> dict:
        """config.json form of this configuration."""
        layers = []
        for l in self.layers:
            m = l.mixer
            if l.type == "retention":
                mixer = dict(heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay), rot=dict(dims=m.rot.dims, base=m.rot.base))
            elif l.type == "parallel":
                left = dict(heads=m.left.heads, kv_heads=m.left.kv_heads, dim=m.left.dim, vdim=m.left.vdim, scale=m.left.scale,
                            conv=m.left.conv, rot=dict(dims=m.left.rot.dims, base=m.left.rot.base))
                if m.left.chunk is not None:
                    left["mask"] = dict(size=m.left.chunk)
                right = dict(heads=m.right.heads, kv_heads=m.right.kv_heads, dim=m.right.dim, vdim=m.right.vdim, conv=m.right.conv)
                if m.right.decay_rank is not None:
                    right["decay_rank"] = m.right.decay_rank
                if m.right.gate_rank is not None:
                    right["gate_rank"] = m.right.gate_rank
                mixer = dict(left=left, right=right)
            else:
                mixer = dict(heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, kv_rank=m.kv_rank, scale=m.scale,
                             rot=dict(dims=m.rot.dims, base=m.rot.base))
                if m.window is not None:
                    mixer["mask"] = dict(size=m.window)
                if m.kv_from is not None:
                    mixer["kv_from"] = m.kv_from
            mlp = None if l.mlp is None else dict(kind="dense", ff=l.mlp.ff, limit=l.mlp.limit)
            layers.append(dict(type=l.type, mixer=mixer, mlp=mlp))
        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, layers=layers, norm=dict(eps=self.norm_eps))
        if self.logit_scale is not None:
            d["logit_scale"] = self.logit_scale
        return d

    def describe(self) -> dict:
        return self.to_dict()
