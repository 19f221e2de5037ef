"""Typed reading of a Kasarax model's config.json.

``layers`` lists the layers one by one: ``type`` names the mixer ("attention"
or "parallel"), ``mixer`` holds its sizes and constants and ``mlp`` the
feed-forward (``kind`` "dense" with ``ff``, or "moe" with ``router``
(``experts``, ``top``) and ``expert`` (``ff``); null for a layer without
one).  An "attention" mixer has ``heads``, ``kv_heads``, ``dim``, ``vdim``,
``scale`` and ``q_temp`` (``coef``, ``every``).  A "parallel" mixer has two
halves: ``left`` (``heads``, ``kv_heads``, ``dim``, ``vdim``, ``scale``,
``conv`` taps, ``rot`` with ``dims`` and ``base``) and ``right`` (``heads``,
``dim``, ``vdim``, one ``decay`` per head).  Model-wide: ``width``, ``vocab``,
``norm.eps`` and ``logit_scale``.  ``architecture`` (a string) names the
design; ``max_position`` is optional (default 2^20: positions are computed,
not tabulated).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

DEFAULT_MAX_POSITION = 1 << 20


def _heads(r: KeyReader):
    heads, kv = r.integer("heads", minimum=1), r.integer("kv_heads", minimum=1)
    if heads % kv:
        raise ConfigError(f"{r.where}: {heads} heads cannot share {kv} key/value heads")
    return heads, kv


@dataclass(frozen=True)
class GatedAttentionConfig:
    """The "attention" mixer: biased projections, a query factor that grows with the logarithm of the position,
    one added to the softmax's denominator, a sigmoid gate per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    temp_coef: float        # the query at position p is multiplied by 1 + coef ln(floor((p + 1) / every) + 1)
    temp_every: int         # 0: no factor

    @staticmethod
    def from_reader(r: KeyReader) -> "GatedAttentionConfig":
        heads, kv = _heads(r)
        temp = r.obj("q_temp")
        return GatedAttentionConfig(
            heads=heads, kv_heads=kv, dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
            scale=r.number("scale", positive=True),
            temp_coef=temp.number("coef") if temp is not None else 0.0,
            temp_every=temp.integer("every", minimum=1) if temp is not None else 0)

    def to_dict(self) -> dict:
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, scale=self.scale, vdim=self.vdim)
        if self.temp_every:
            d["q_temp"] = dict(coef=self.temp_coef, every=self.temp_every)
        return d


@dataclass(frozen=True)
class ConvAttentionConfig:
    """The left half of a "parallel" mixer: convolutions on q, k and v, norms over the whole of q and of k,
    interleaved rotation of part of a head, a learned sink per head."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    conv: int               # taps of the convolutions (1: a factor per channel on the current token; 0: none)
    rot_dims: int
    rot_base: float

    @staticmethod
    def from_reader(r: KeyReader) -> "ConvAttentionConfig":
        heads, kv = _heads(r)
        dim = r.integer("dim", minimum=1)
        rot = r.obj("rot")
        dims = rot.integer("dims", minimum=0) if rot is not None else 0
        base = rot.number("base", positive=True) if rot is not None else 10000.0
        if dims % 2 or dims > dim:
            raise ConfigError(f"{r.where}: rot.dims {dims} must be even and at most dim {dim}")
        return ConvAttentionConfig(heads=heads, kv_heads=kv, dim=dim, vdim=r.integer("vdim", minimum=1),
                                   scale=r.number("scale", positive=True), conv=r.integer("conv", 0, minimum=0),
                                   rot_dims=dims, rot_base=base)

    def to_dict(self) -> dict:
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, scale=self.scale, vdim=self.vdim)
        if self.conv:
            d["conv"] = self.conv
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
        return d


@dataclass(frozen=True)
class LightningConfig:
    """The right half of a "parallel" mixer: linear attention with a fixed decay per head."""
    heads: int
    dim: int
    vdim: int
    decay: tuple            # one per head

    @staticmethod
    def from_reader(r: KeyReader) -> "LightningConfig":
        c = LightningConfig(heads=r.integer("heads", minimum=1), dim=r.integer("dim", minimum=1),
                            vdim=r.integer("vdim", minimum=1), decay=r.number_list("decay"))
        if len(c.decay) != c.heads:
            raise ConfigError(f"{r.where}: {len(c.decay)} decays for {c.heads} heads")
        return c

    def to_dict(self) -> dict:
        return dict(decay=list(self.decay), dim=self.dim, heads=self.heads, vdim=self.vdim)


@dataclass(frozen=True)
class PairConfig:
    left: ConvAttentionConfig
    right: LightningConfig

    @staticmethod
    def from_reader(r: KeyReader) -> "PairConfig":
        left, right = r.obj("left"), r.obj("right")
        if left is None or right is None:
            raise ConfigError(f"{r.where}: 'left' and 'right' are required")
        return PairConfig(ConvAttentionConfig.from_reader(left), LightningConfig.from_reader(right))

    def to_dict(self) -> dict:
        return dict(left=self.left.to_dict(), right=self.right.to_dict())


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str               # "dense" or "moe"
    ff: int                 # inner size (of one expert, for "moe")
    experts: int = 0
    top: int = 0

    @staticmethod
    def from_reader(r: KeyReader) -> "FeedForwardConfig":
        kind = r.string("kind")
        if kind == "dense":
            return FeedForwardConfig("dense", r.integer("ff", minimum=1))
        if kind != "moe":
            raise ConfigError(f"{r.where}: feed-forward kind {kind!r} is not known; known: ['dense', 'moe']")
        router, expert = r.obj("router"), r.obj("expert")
        if router is None or expert is None:
            raise ConfigError(f"{r.where}: 'router' and 'expert' are required")
        c = FeedForwardConfig("moe", expert.integer("ff", minimum=1), experts=router.integer("experts", minimum=1),
                              top=router.integer("top", minimum=1))
        if c.top > c.experts:
            raise ConfigError(f"{r.where}: top {c.top} is more than the {c.experts} experts")
        return c

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return dict(ff=self.ff, kind="dense")
        return dict(expert=dict(ff=self.ff), kind="moe", router=dict(experts=self.experts, top=self.top))


_MIXERS = {"attention": GatedAttentionConfig, "parallel": PairConfig}


@dataclass(frozen=True)
class KasaraxLayerConfig:
    type: str
    mixer: object
    mlp: FeedForwardConfig | None

    @staticmethod
    def from_reader(r: KeyReader) -> "KasaraxLayerConfig":
        kind = r.string("type")
        if kind not in _MIXERS:
            raise ConfigError(f"{r.where}: layer type {kind!r} is not known; known: {sorted(_MIXERS)}")
        mixer, mlp = r.obj("mixer"), r.obj("mlp")
        if mixer is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        return KasaraxLayerConfig(kind, _MIXERS[kind].from_reader(mixer),
                                  FeedForwardConfig.from_reader(mlp) if mlp is not None else None)

    def to_dict(self) -> dict:
        return dict(mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None, type=self.type)


@dataclass
class KasaraxConfig:
    architecture: str
    width: int
    vocab: int
    layers: tuple
    norm_eps: float
    logit_scale: float = 1.0
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_id: tuple = field(default_factory=tuple)

    ARCHITECTURE = "Kasarax"

    @staticmethod
    def from_dict(data: dict, where: str = "config.json") -> "KasaraxConfig":
        r = KeyReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(KasaraxLayerConfig.from_reader(KeyReader(x, f"{where}:layers[{i}]"))
                       for i, x in enumerate(raw_layers))
        norm = r.obj("norm")
        if norm is None:
            raise ConfigError(f"{where}: required key 'norm' is missing")
        return KasaraxConfig(
            architecture=r.string("architecture", KasaraxConfig.ARCHITECTURE),
            width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), layers=layers,
            norm_eps=norm.number("eps", positive=True), logit_scale=r.number("logit_scale", 1.0),
            max_position=r.integer("max_position", DEFAULT_MAX_POSITION, minimum=1),
            eos_token_id=r.int_list("eos_token_id", ()))

    def to_dict(self) -> dict:
        d = dict(architecture=self.architecture, layers=[x.to_dict() for x in self.layers],
                 logit_scale=self.logit_scale, norm=dict(eps=self.norm_eps), vocab=self.vocab, width=self.width)
        if self.max_position != DEFAULT_MAX_POSITION:
            d["max_position"] = self.max_position
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
