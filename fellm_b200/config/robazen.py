"""Typed configuration of the Robazen design, read from its config.json.

The file is nested: `layers` is a list of {type, mixer, mlp}, `loop` = {start, stop, times} names a
run of layers that is repeated with the same weights, `norm` = {eps}.  Every size and every constant
that can differ between two models of the design is read here; a missing or ill-typed key raises
ConfigError with the key's path.  FeLLM keeps such facts in its probed `ModelSpec`
(crates/fellm-model/src/probe.rs:86-181); it has no nested layer list.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional

from .errors import ConfigError

NAME = "Robazen"
LAYER_TYPES = ("delta", "channel_delta", "parallel")


def _get(d, key, kind, where, *, default=None, required=True, positive=False):
    if not isinstance(d, dict):
        raise ConfigError(f"config.json: {where} must be an object")
    if key not in d or d[key] is None:
        if required:
            raise ConfigError(f"config.json: missing key '{where}.{key}'" if where else f"config.json: missing key '{key}'")
        return default
    v = d[key]
    if kind is int:
        if isinstance(v, bool) or not isinstance(v, int):
            raise ConfigError(f"config.json: '{where}.{key}' must be an integer, got {v!r}")
        if positive and v < 1:
            raise ConfigError(f"config.json: '{where}.{key}' must be positive, got {v}")
        return int(v)
    if kind is float:
        if isinstance(v, bool) or not isinstance(v, (int, float)):
            raise ConfigError(f"config.json: '{where}.{key}' must be a number, got {v!r}")
        return float(v)
    if kind is dict:
        if not isinstance(v, dict):
            raise ConfigError(f"config.json: '{where}.{key}' must be an object")
        return v
    return v


@dataclass(frozen=True)
class DeltaMixerConfig:
    """Sizes of a gated-delta-rule mixer ('delta' and 'channel_delta')."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    conv: int

    @staticmethod
    def read(d, where):
        c = DeltaMixerConfig(heads=_get(d, "heads", int, where, positive=True),
                             kv_heads=_get(d, "kv_heads", int, where, positive=True),
                             dim=_get(d, "dim", int, where, positive=True),
                             vdim=_get(d, "vdim", int, where, positive=True),
                             conv=_get(d, "conv", int, where, positive=True))
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' ({c.heads}) is not a multiple of kv_heads ({c.kv_heads})")
        return c

    def to_dict(self):
        return dict(conv=self.conv, dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, vdim=self.vdim)


@dataclass(frozen=True)
class ChunkAttentionConfig:
    """The softmax-attention half of a 'parallel' mixer."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    softcap: Optional[float]
    chunk: int

    @staticmethod
    def read(d, where):
        mask = _get(d, "mask", dict, where)
        c = ChunkAttentionConfig(heads=_get(d, "heads", int, where, positive=True),
                                 kv_heads=_get(d, "kv_heads", int, where, positive=True),
                                 dim=_get(d, "dim", int, where, positive=True),
                                 vdim=_get(d, "vdim", int, where, positive=True),
                                 scale=_get(d, "scale", float, where),
                                 softcap=_get(d, "softcap", float, where, required=False),
                                 chunk=_get(mask, "size", int, where + ".mask", positive=True))
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' ({c.heads}) is not a multiple of kv_heads ({c.kv_heads})")
        if c.softcap is not None and c.softcap <= 0:
            raise ConfigError(f"config.json: '{where}.softcap' must be positive, got {c.softcap}")
        return c

    def to_dict(self):
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, mask=dict(size=self.chunk),
                 scale=self.scale, vdim=self.vdim)
        if self.softcap is not None:
            d["softcap"] = self.softcap
        return d


@dataclass(frozen=True)
class TimeMixConfig:
    """The recurrent half of a 'parallel' mixer."""
    heads: int
    dim: int

    @staticmethod
    def read(d, where):
        return TimeMixConfig(heads=_get(d, "heads", int, where, positive=True),
                             dim=_get(d, "dim", int, where, positive=True))

    def to_dict(self):
        return dict(dim=self.dim, heads=self.heads)


@dataclass(frozen=True)
class ParallelMixerConfig:
    left: ChunkAttentionConfig
    right: TimeMixConfig

    def to_dict(self):
        return dict(left=self.left.to_dict(), right=self.right.to_dict())


@dataclass(frozen=True)
class RobazenLayer:
    type: str
    mixer: object
    ff: Optional[int]            # None: the layer has no feed-forward

    def to_dict(self):
        return dict(mixer=self.mixer.to_dict(), mlp=None if self.ff is None else dict(ff=self.ff, kind="dense"),
                    type=self.type)


@dataclass(frozen=True)
class LoopConfig:
    start: int
    stop: int
    times: int


@dataclass
class RobazenConfig:
    vocab: int
    width: int
    norm_eps: float
    layers: List[RobazenLayer] = field(default_factory=list)
    loop: Optional[LoopConfig] = None

    @staticmethod
    def from_dict(d: dict) -> "RobazenConfig":
        vocab = _get(d, "vocab", int, "", positive=True)
        width = _get(d, "width", int, "", positive=True)
        eps = _get(_get(d, "norm", dict, ""), "eps", float, "norm")
        raw = d.get("layers")
        if not isinstance(raw, list) or not raw:
            raise ConfigError("config.json: 'layers' must be a non-empty list")
        layers = []
        for i, L in enumerate(raw):
            where = f"layers[{i}]"
            kind = _get(L, "type", str, where)
            if kind not in LAYER_TYPES:
                raise ConfigError(f"config.json: '{where}.type' is {kind!r}; known: {', '.join(LAYER_TYPES)}")
            m = _get(L, "mixer", dict, where)
            if kind == "parallel":
                mixer = ParallelMixerConfig(ChunkAttentionConfig.read(_get(m, "left", dict, where + ".mixer"), where + ".mixer.left"),
                                            TimeMixConfig.read(_get(m, "right", dict, where + ".mixer"), where + ".mixer.right"))
            else:
                mixer = DeltaMixerConfig.read(m, where + ".mixer")
            mlp = L.get("mlp")
            ff = None
            if mlp is not None:
                mkind = _get(mlp, "kind", str, where + ".mlp")
                if mkind != "dense":
                    raise ConfigError(f"config.json: '{where}.mlp.kind' is {mkind!r}; known: dense")
                ff = _get(mlp, "ff", int, where + ".mlp", positive=True)
            layers.append(RobazenLayer(kind, mixer, ff))
        loop = None
        if d.get("loop") is not None:
            lp = _get(d, "loop", dict, "")
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"),
                              _get(lp, "times", int, "loop", positive=True))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: 'loop' names layers {loop.start}..{loop.stop - 1} of {len(layers)}")
        return RobazenConfig(vocab=vocab, width=width, norm_eps=eps, layers=layers, loop=loop)

    def to_dict(self) -> dict:
        d = dict(architecture=NAME, layers=[L.to_dict() for L in self.layers], norm=dict(eps=self.norm_eps),
                 vocab=self.vocab, width=self.width)
        if self.loop is not None:
            d["loop"] = dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times)
        return d
