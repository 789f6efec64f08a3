"""Configuration of the Rutetar design (config.json "architecture": "Rutetar").

A decoder whose layers are listed one by one: each entry of `layers` names its mixer (`type`), the mixer's sizes (`mixer`)
and its feed-forward (`mlp`, or null).  Mixer 'retention' is linear attention with a fixed decay per head; mixer 'parallel'
runs two mixers side by side on the same input, softmax attention in a sliding window with an output gate per head
(`left`) and time mixing with a decay per token and channel (`right`), and adds them with two scales.  The feed-forward is
dense and gated, or a mixture of gated experts.  A stretch of layers may run several times in a row (`loop`), and the
residual is kept as several streams (`streams`).  Every size and every constant that can differ between two models of the
design is read here; nothing of them stands in code.
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, ConfigReader

ARCHITECTURE = "Rutetar"
MIXERS = ("retention", "parallel")
MLP_KINDS = ("dense", "moe")


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int                 # per head: query/key entries
    vdim: int                # per head: value entries
    decay: tuple             # one constant per head


@dataclass(frozen=True)
class WindowAttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: int | None       # positions that a token sees, itself included; None: all before it
    rot_dims: int            # rotated entries of every head (the first ones), even; 0: none
    rot_base: float


@dataclass(frozen=True)
class TimeMixConfig:
    heads: int
    dim: int
    rank: int | None         # width of the decay's inner projection; None: whatever the checkpoint's tensors hold


@dataclass(frozen=True)
class ParallelConfig:
    left: WindowAttentionConfig
    right: TimeMixConfig
    left_scale: float
    right_scale: float


@dataclass(frozen=True)
class MlpConfig:
    kind: str                # "dense" or "moe"
    ff: int                  # inner width (of an expert, for "moe")
    experts: int = 0
    top: int = 0


@dataclass(frozen=True)
class LayerConfig:
    type: str
    mixer: object            # RetentionConfig or ParallelConfig
    mlp: MlpConfig | None


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass(frozen=True)
class RutetarConfig:
    vocab: int
    width: int
    layers: tuple
    norm_eps: float
    streams: int | None      # None: one residual without mixing tables
    loop: LoopConfig | None
    raw: dict = field(compare=False, repr=False, default_factory=dict)

    architecture = ARCHITECTURE

    @classmethod
    def from_dict(cls, data: dict, source: str = "config.json") -> "RutetarConfig":
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
                heads = e.integer("mixer.heads", minimum=1)
                decay = entry["mixer"].get("decay")
                if not isinstance(decay, list) or len(decay) != heads or \
                        not all(isinstance(d, (int, float)) and not isinstance(d, bool) for d in decay):
                    raise ConfigError(f"{where}: mixer.decay must be a list of {heads} numbers, one per head")
                mixer = RetentionConfig(heads=heads, dim=e.integer("mixer.dim", minimum=1), vdim=e.integer("mixer.vdim", minimum=1),
                                        decay=tuple(float(d) for d in decay))
            else:
                dim = e.integer("mixer.left.dim", minimum=1)
                left = WindowAttentionConfig(
                    heads=e.integer("mixer.left.heads", minimum=1), kv_heads=e.integer("mixer.left.kv_heads", minimum=1), dim=dim,
                    vdim=e.integer("mixer.left.vdim", minimum=1), scale=e.number("mixer.left.scale", exclusive_minimum=0.0),
                    window=e.integer("mixer.left.mask.size", default=None, minimum=1),
                    rot_dims=e.integer("mixer.left.rot.dims", default=0, minimum=0),
                    rot_base=e.number("mixer.left.rot.base", default=10000.0, exclusive_minimum=0.0))
                if left.heads % left.kv_heads:
                    raise ConfigError(f"{where}: mixer.left.heads {left.heads} is not a multiple of mixer.left.kv_heads {left.kv_heads}")
                if left.rot_dims % 2 or left.rot_dims > dim:
                    raise ConfigError(f"{where}: mixer.left.rot.dims {left.rot_dims} must be even and at most mixer.left.dim {dim}")
                right = TimeMixConfig(heads=e.integer("mixer.right.heads", minimum=1), dim=e.integer("mixer.right.dim", minimum=1),
                                      rank=e.integer("mixer.right.rank", default=None, minimum=1))
                mixer = ParallelConfig(left=left, right=right, left_scale=e.number("mixer.left_scale"),
                                       right_scale=e.number("mixer.right_scale"))
            mlp = None
            if entry.get("mlp") is not None:
                mlp_kind = e.string("mlp.kind")
                if mlp_kind not in MLP_KINDS:
                    raise ConfigError(f"{where}: mlp.kind '{mlp_kind}' is not known (known: {', '.join(MLP_KINDS)})")
                if mlp_kind == "dense":
                    mlp = MlpConfig("dense", ff=e.integer("mlp.ff", minimum=1))
                else:
                    mlp = MlpConfig("moe", ff=e.integer("mlp.expert.ff", minimum=1), experts=e.integer("mlp.router.experts", minimum=1),
                                    top=e.integer("mlp.router.top", minimum=1))
                    if mlp.top > mlp.experts:
                        raise ConfigError(f"{where}: mlp.router.top {mlp.top} is more than mlp.router.experts {mlp.experts}")
            layers.append(LayerConfig(kind, mixer, mlp))
        loop = None
        if data.get("loop") is not None:
            loop = LoopConfig(start=r.integer("loop.start", minimum=0), stop=r.integer("loop.stop", minimum=0),
                              times=r.integer("loop.times", minimum=1))
            if not (loop.start <= loop.stop <= len(layers)):
                raise ConfigError(f"{source}: loop.start {loop.start} and loop.stop {loop.stop} must lie in order within the {len(layers)} layers")
        return cls(vocab=r.integer("vocab", minimum=1), width=width, layers=tuple(layers),
                   norm_eps=r.number("norm.eps", exclusive_minimum=0.0), streams=r.integer("streams", default=None, minimum=1),
                   loop=loop, raw=data)

    def order(self) -> list:
        """The layers in the order they run: those of the loop `times` times in a row, the others once."""
        n = len(self.layers)
        if self.loop is None:
            return list(range(n))
        a, b = self.loop.start, self.loop.stop
        return list(range(a)) + list(range(a, b)) * self.loop.times + list(range(b, n))

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
                mixer = dict(heads=m.heads, dim=m.dim, vdim=m.vdim, decay=list(m.decay))
            else:
                left = dict(heads=m.left.heads, kv_heads=m.left.kv_heads, dim=m.left.dim, vdim=m.left.vdim, scale=m.left.scale,
                            rot=dict(dims=m.left.rot_dims, base=m.left.rot_base))
                if m.left.window is not None:
                    left["mask"] = dict(size=m.left.window)
                right = dict(heads=m.right.heads, dim=m.right.dim)
                if m.right.rank is not None:
                    right["rank"] = m.right.rank
                mixer = dict(left=left, right=right, left_scale=m.left_scale, right_scale=m.right_scale)
            mlp = None
            if l.mlp is not None:
                mlp = dict(kind="dense", ff=l.mlp.ff) if l.mlp.kind == "dense" else \
                    dict(kind="moe", expert=dict(ff=l.mlp.ff), router=dict(experts=l.mlp.experts, top=l.mlp.top))
            layers.append(dict(type=l.type, mixer=mixer, mlp=mlp))
        d = dict(architecture=ARCHITECTURE, vocab=self.vocab, width=self.width, layers=layers, norm=dict(eps=self.norm_eps))
        if self.streams is not None:
            d["streams"] = self.streams
        if self.loop is not None:
            d["loop"] = dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times)
        return d

    def describe(self) -> dict:
        return self.to_dict()
