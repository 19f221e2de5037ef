"""Typed reading of a Mepatar model's config.json.

``layers`` lists the layers one by one: ``type`` names the mixer ("retention",
"attention" or "delta"), ``mixer`` holds its sizes and constants and ``mlp``
the feed-forward (``kind`` "dense" with ``ff``, or "moe" with ``router``
(``experts``, ``top``) and ``expert`` (``ff``, ``limit``); null for a layer
without one).  Model-wide: ``width``, ``vocab``, ``norm`` (``eps``, ``groups``:
the parts a row is cut into, each normed on its own), ``embedding.scale``
(the factor on the embedding rows) and ``canon.taps`` (the length of the
causal convolution in front of every mixer; absent or 0: none).
``architecture`` (a string) names the design; ``max_position`` is optional
(default 2^20: positions are computed, not tabulated).
"""
from __future__ import annotations

from dataclasses import dataclass, field

from .base import ConfigError, KeyReader

DEFAULT_MAX_POSITION = 1 << 20


def _rotation(r: KeyReader, limit: int):
    """(dims, base) of a mixer's ``rot`` object; no object means no rotation."""
    rot = r.obj("rot")
    if rot is None:
        return 0, 10000.0
    dims, base = rot.integer("dims", minimum=0), rot.number("base", positive=True)
    if dims % 2 or dims > limit:
        raise ConfigError(f"{r.where}: rot.dims {dims} must be even and at most dim {limit}")
    return dims, base


@dataclass(frozen=True)
class RetentionConfig:
    heads: int
    dim: int
    vdim: int
    decay: tuple            # one per head
    rot_dims: int
    rot_base: float

    @staticmethod
    def from_reader(r: KeyReader) -> "RetentionConfig":
        dim = r.integer("dim", minimum=1)
        dims, base = _rotation(r, dim)
        c = RetentionConfig(heads=r.integer("heads", minimum=1), dim=dim, vdim=r.integer("vdim", minimum=1),
                            decay=r.number_list("decay"), rot_dims=dims, rot_base=base)
        if len(c.decay) != c.heads:
            raise ConfigError(f"{r.where}: {len(c.decay)} decays for {c.heads} heads")
        return c

    def to_dict(self) -> dict:
        d = dict(decay=list(self.decay), dim=self.dim, heads=self.heads, vdim=self.vdim)
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
        return d


@dataclass(frozen=True)
class AttentionConfig:
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    rot_dims: int
    rot_base: float
    window: int             # positions a query sees, itself included (0: all before it)
    keep_first: int         # the first positions that stay visible whatever the window

    @staticmethod
    def from_reader(r: KeyReader) -> "AttentionConfig":
        dim = r.integer("dim", minimum=1)
        dims, base = _rotation(r, dim)
        mask = r.obj("mask")
        c = AttentionConfig(
            heads=r.integer("heads", minimum=1), kv_heads=r.integer("kv_heads", minimum=1), dim=dim,
            vdim=r.integer("vdim", minimum=1), scale=r.number("scale", positive=True), rot_dims=dims, rot_base=base,
            window=mask.integer("size", 0, minimum=0) if mask is not None else 0,
            keep_first=mask.integer("keep_first", 0, minimum=0) if mask is not None else 0)
        if c.heads % c.kv_heads:
            raise ConfigError(f"{r.where}: {c.heads} heads cannot share {c.kv_heads} key/value heads")
        return c

    def to_dict(self) -> dict:
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, scale=self.scale, vdim=self.vdim)
        if self.rot_dims:
            d["rot"] = dict(base=self.rot_base, dims=self.rot_dims)
        if self.window:
            d["mask"] = dict(keep_first=self.keep_first, size=self.window)
        return d


@dataclass(frozen=True)
class DeltaConfig:
    heads: int
    kv_heads: int           # query/key heads
    dim: int
    vdim: int
    conv: int               # taps of the convolutions on q, k and v

    @staticmethod
    def from_reader(r: KeyReader) -> "DeltaConfig":
        c = DeltaConfig(heads=r.integer("heads", minimum=1), kv_heads=r.integer("kv_heads", minimum=1),
                        dim=r.integer("dim", minimum=1), vdim=r.integer("vdim", minimum=1),
                        conv=r.integer("conv", minimum=1))
        if c.heads % c.kv_heads:
            raise ConfigError(f"{r.where}: {c.heads} heads cannot share {c.kv_heads} query/key heads")
        return c

    def to_dict(self) -> dict:
        return dict(conv=self.conv, dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, vdim=self.vdim)


@dataclass(frozen=True)
class FeedForwardConfig:
    kind: str               # "dense" or "moe"
    ff: int                 # inner size (of one expert, for "moe")
    experts: int = 0
    top: int = 0
    limit: float = 0.0

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
                              top=router.integer("top", minimum=1), limit=expert.number("limit", positive=True))
        if c.top > c.experts:
            raise ConfigError(f"{r.where}: top {c.top} is more than the {c.experts} experts")
        return c

    def to_dict(self) -> dict:
        if self.kind == "dense":
            return dict(ff=self.ff, kind="dense")
        return dict(expert=dict(ff=self.ff, limit=self.limit), kind="moe",
                    router=dict(experts=self.experts, top=self.top))


_MIXERS = {"retention": RetentionConfig, "attention": AttentionConfig, "delta": DeltaConfig}


@dataclass(frozen=True)
class MepatarLayerConfig:
    type: str
    mixer: object
    mlp: FeedForwardConfig | None

    @staticmethod
    def from_reader(r: KeyReader) -> "MepatarLayerConfig":
        kind = r.string("type")
        if kind not in _MIXERS:
            raise ConfigError(f"{r.where}: layer type {kind!r} is not known; known: {sorted(_MIXERS)}")
        mixer, mlp = r.obj("mixer"), r.obj("mlp")
        if mixer is None:
            raise ConfigError(f"{r.where}: required key 'mixer' is missing")
        return MepatarLayerConfig(kind, _MIXERS[kind].from_reader(mixer),
                                  FeedForwardConfig.from_reader(mlp) if mlp is not None else None)

    def to_dict(self) -> dict:
        return dict(mixer=self.mixer.to_dict(), mlp=self.mlp.to_dict() if self.mlp else None, type=self.type)


@dataclass
class MepatarConfig:
    architecture: str
    width: int
    vocab: int
    layers: tuple
    norm_eps: float
    norm_groups: int = 1
    embedding_scale: float = 1.0
    canon_taps: int = 0
    max_position: int = DEFAULT_MAX_POSITION
    eos_token_id: tuple = field(default_factory=tuple)

    ARCHITECTURE = "Mepatar"

    @staticmethod
    def from_dict(data: dict, where: str = "config.json") -> "MepatarConfig":
        r = KeyReader(data, where)
        raw_layers = data.get("layers")
        if not isinstance(raw_layers, list) or not raw_layers:
            raise ConfigError(f"{where}: 'layers' must be a non-empty list")
        layers = tuple(MepatarLayerConfig.from_reader(KeyReader(x, f"{where}:layers[{i}]"))
                       for i, x in enumerate(raw_layers))
        norm = r.obj("norm")
        if norm is None:
            raise ConfigError(f"{where}: required key 'norm' is missing")
        emb, canon = r.obj("embedding"), r.obj("canon")
        c = MepatarConfig(
            architecture=r.string("architecture", MepatarConfig.ARCHITECTURE),
            width=r.integer("width", minimum=1), vocab=r.integer("vocab", minimum=1), layers=layers,
            norm_eps=norm.number("eps", positive=True), norm_groups=norm.integer("groups", 1, minimum=1),
            embedding_scale=emb.number("scale", 1.0) if emb is not None else 1.0,
            canon_taps=canon.integer("taps", 0, minimum=0) if canon is not None else 0,
            max_position=r.integer("max_position", DEFAULT_MAX_POSITION, minimum=1),
            eos_token_id=r.int_list("eos_token_id", ()))
        if c.width % c.norm_groups:
            raise ConfigError(f"{where}: width {c.width} does not split into {c.norm_groups} equal norm groups")
        return c

    def to_dict(self) -> dict:
        d = dict(architecture=self.architecture, embedding=dict(scale=self.embedding_scale),
                 layers=[x.to_dict() for x in self.layers], norm=dict(eps=self.norm_eps, groups=self.norm_groups),
                 vocab=self.vocab, width=self.width)
        if self.canon_taps:
            d["canon"] = dict(taps=self.canon_taps)
        if self.max_position != DEFAULT_MAX_POSITION:
            d["max_position"] = self.max_position
        if self.eos_token_id:
            d["eos_token_id"] = list(self.eos_token_id)
        return d
