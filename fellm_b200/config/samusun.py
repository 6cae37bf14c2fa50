"""Typed configuration of the Samusun design, read from its config.json.

The file is nested like Robazen's: `layers` is a list of {type, mixer, mlp}, `loop` = {start, stop, times} names a
run of layers that is repeated with the same weights, `norm` = {eps}; beside those `embedding.scale`,
`logit_scale`, `logit_softcap`.  A layer's `type` is 'attention' or 'retention'; its `mlp` is null, a dense
feed-forward {kind: dense, ff} or routed experts {kind: moe, expert: {ff}, router: {experts, top}}.  Every size and
every constant that can differ between two models of the design is read here; a missing or ill-typed key raises
ConfigError with the key's path.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import List, Optional, Tuple

from .errors import ConfigError
from .robazen import LoopConfig, _get

NAME = "Samusun"
LAYER_TYPES = ("attention", "retention")


@dataclass(frozen=True)
class WindowAttentionConfig:
    """The 'attention' mixer: the keys are also the values, a sliding window, a query temperature by position."""
    heads: int
    kv_heads: int
    dim: int
    vdim: int
    scale: float
    window: Optional[int]
    q_temp_coef: float
    q_temp_every: int

    @staticmethod
    def read(d, where):
        # a file that leaves out the window or the temperature has none; kv_heads defaults to heads
        mask = _get(d, "mask", dict, where, required=False)
        qt = _get(d, "q_temp", dict, where, required=False)
        heads = _get(d, "heads", int, where, positive=True)
        dim = _get(d, "dim", int, where, positive=True)
        c = WindowAttentionConfig(heads=heads,
                                  kv_heads=_get(d, "kv_heads", int, where, positive=True, required=False, default=heads),
                                  dim=dim,
                                  vdim=_get(d, "vdim", int, where, positive=True, required=False, default=dim),
                                  scale=_get(d, "scale", float, where),
                                  window=None if mask is None else _get(mask, "size", int, where + ".mask", positive=True),
                                  q_temp_coef=0.0 if qt is None else _get(qt, "coef", float, where + ".q_temp"),
                                  q_temp_every=0 if qt is None else _get(qt, "every", int, where + ".q_temp", positive=True))
        if c.heads % c.kv_heads:
            raise ConfigError(f"config.json: '{where}.heads' ({c.heads}) is not a multiple of kv_heads ({c.kv_heads})")
        if c.vdim != c.dim:
            raise ConfigError(f"config.json: '{where}.vdim' ({c.vdim}) must equal dim ({c.dim}): the values are the keys")
        return c

    def to_dict(self):
        d = dict(dim=self.dim, heads=self.heads, kv_heads=self.kv_heads, scale=self.scale, vdim=self.vdim)
        if self.window is not None:
            d["mask"] = dict(size=self.window)
        if self.q_temp_every:
            d["q_temp"] = dict(coef=self.q_temp_coef, every=self.q_temp_every)
        return d


@dataclass(frozen=True)
class RetentionConfig:
    """The 'retention' mixer: a decaying sum of k v^T per head, rotary positions on part of q and k."""
    heads: int
    dim: int
    vdim: int
    decay: Tuple[float, ...]
    rot_dims: int
    rot_base: float

    @staticmethod
    def read(d, where):
        rot = _get(d, "rot", dict, where, required=False)          # left out: no rotation
        decay = d.get("decay")
        if not isinstance(decay, list) or any(isinstance(g, bool) or not isinstance(g, (int, float)) for g in decay):
            raise ConfigError(f"config.json: '{where}.decay' must be a list of numbers")
        c = RetentionConfig(heads=_get(d, "heads", int, where, positive=True),
                            dim=_get(d, "dim", int, where, positive=True),
                            vdim=_get(d, "vdim", int, where, positive=True),
                            decay=tuple(float(g) for g in decay),
                            rot_dims=0 if rot is None else _get(rot, "dims", int, where + ".rot"),
                            rot_base=10000.0 if rot is None else _get(rot, "base", float, where + ".rot"))
        if len(c.decay) != c.heads:
            raise ConfigError(f"config.json: '{where}.decay' has {len(c.decay)} entries for {c.heads} heads")
        if c.rot_dims % 2 or not 0 <= c.rot_dims <= c.dim:
            raise ConfigError(f"config.json: '{where}.rot.dims' ({c.rot_dims}) must be even and at most dim ({c.dim})")
        if c.rot_base <= 0:
            raise ConfigError(f"config.json: '{where}.rot.base' must be positive, got {c.rot_base}")
        return c

    def to_dict(self):
        return dict(decay=list(self.decay), dim=self.dim, heads=self.heads, rot=dict(base=self.rot_base, dims=self.rot_dims),
                    vdim=self.vdim)


@dataclass(frozen=True)
class FeedForwardConfig:
    """kind 'dense': one gated feed-forward of `ff`; 'moe': `experts` of them, each of `ff`, `top` a token."""
    kind: str
    ff: int
    experts: int = 0
    top: int = 0

    @staticmethod
    def read(d, where):
        kind = _get(d, "kind", str, where)
        if kind == "dense":
            return FeedForwardConfig("dense", _get(d, "ff", int, where, positive=True))
        if kind == "moe":
            router = _get(d, "router", dict, where)
            c = FeedForwardConfig("moe", _get(_get(d, "expert", dict, where), "ff", int, where + ".expert", positive=True),
                                  _get(router, "experts", int, where + ".router", positive=True),
                                  _get(router, "top", int, where + ".router", positive=True))
            if c.top > c.experts:
                raise ConfigError(f"config.json: '{where}.router.top' ({c.top}) is above experts ({c.experts})")
            return c
        raise ConfigError(f"config.json: '{where}.kind' is {kind!r}; known: dense, moe")

    def to_dict(self):
        if self.kind == "dense":
            return dict(ff=self.ff, kind="dense")
        return dict(expert=dict(ff=self.ff), kind="moe", router=dict(experts=self.experts, top=self.top))


@dataclass(frozen=True)
class SamusunLayer:
    type: str
    mixer: object
    mlp: Optional[FeedForwardConfig]          # None: the layer has no feed-forward

    def to_dict(self):
        return dict(mixer=self.mixer.to_dict(), mlp=None if self.mlp is None else self.mlp.to_dict(), type=self.type)


@dataclass
class SamusunConfig:
    vocab: int
    width: int
    norm_eps: float
    embedding_scale: float = 1.0
    logit_scale: float = 1.0
    logit_softcap: Optional[float] = None
    layers: List[SamusunLayer] = field(default_factory=list)
    loop: Optional[LoopConfig] = None

    @staticmethod
    def from_dict(d: dict) -> "SamusunConfig":
        vocab = _get(d, "vocab", int, "", positive=True)
        width = _get(d, "width", int, "", positive=True)
        eps = _get(_get(d, "norm", dict, ""), "eps", float, "norm")
        emb = _get(d, "embedding", dict, "", required=False, default={})
        emb_scale = _get(emb, "scale", float, "embedding", required=False, default=1.0)
        logit_scale = _get(d, "logit_scale", float, "", required=False, default=1.0)
        cap = _get(d, "logit_softcap", float, "", required=False)
        if cap is not None and cap <= 0:
            raise ConfigError(f"config.json: 'logit_softcap' must be positive, got {cap}")
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
            mixer = (WindowAttentionConfig if kind == "attention" else RetentionConfig).read(m, where + ".mixer")
            mlp = None if L.get("mlp") is None else FeedForwardConfig.read(L["mlp"], where + ".mlp")
            layers.append(SamusunLayer(kind, mixer, mlp))
        loop = None
        if d.get("loop") is not None:
            lp = _get(d, "loop", dict, "")
            loop = LoopConfig(_get(lp, "start", int, "loop"), _get(lp, "stop", int, "loop"),
                              _get(lp, "times", int, "loop", positive=True))
            if not 0 <= loop.start < loop.stop <= len(layers):
                raise ConfigError(f"config.json: 'loop' names layers {loop.start}..{loop.stop - 1} of {len(layers)}")
        return SamusunConfig(vocab=vocab, width=width, norm_eps=eps, embedding_scale=emb_scale, logit_scale=logit_scale,
                             logit_softcap=cap, layers=layers, loop=loop)

    def to_dict(self) -> dict:
        d = dict(architecture=NAME, embedding=dict(scale=self.embedding_scale), layers=[L.to_dict() for L in self.layers],
                 logit_scale=self.logit_scale, norm=dict(eps=self.norm_eps), vocab=self.vocab, width=self.width)
        if self.logit_softcap is not None:
            d["logit_softcap"] = self.logit_softcap
        if self.loop is not None:
            d["loop"] = dict(start=self.loop.start, stop=self.loop.stop, times=self.loop.times)
        return d
