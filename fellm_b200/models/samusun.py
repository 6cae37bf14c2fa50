"""Samusun: how the design is put together from parts.

A layer is `h = norm1(x); x += mixer(h) + ff(h)`: one RMS norm, mixer and feed-forward side by side (the
'parallel' arrangement); a layer may have no feed-forward.  A layer's mixer is one of
  attention   softmax attention whose values are its keys (no W_v; the cache keeps keys alone), biased q, k and
              output projections, no rotation, a query temperature by position, a bias by distance with slopes
              2^(-8 (h + 1) / H), a sliding window                                          (parts/attention.py)
  retention   a decaying sum of k v^T per head with a fixed decay, rotary positions on part of q and k, the read-out
              over its root mean square per head, a SiLU gate                               (parts/retention.py)
and its feed-forward W_down(SiLU(W_gate h) * W_up h), dense (parts/swiglu.py) or as routed experts (parts/moe.py:
softmax scores over all experts, the `top` largest, weighted by their scores as they are).  `loop` repeats a run of
layers with the same weights, each pass with caches and states of its own; a pass opens with x <- x + step[t]
(parts/connector.py, 'add_step').  The embedding is scaled; the logits are scaled and soft-capped.

Tensor names of the safetensors file: embed, head, final.norm, loop.step, and per layer i: l<i>.norm1,
l<i>.mix.{q,k,o}{,.b} (attention) or l<i>.mix.{q,k,v,g,o} (retention), l<i>.mlp.{gate,up,down} (dense) or
l<i>.mlp.router and l<i>.mlp.e<j>.{gate,up,down} (experts).
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.samusun import NAME, SamusunConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20        # nothing ends a context but memory: windows slide and states have a fixed size
SLOPE_EXP = 8.0               # the design's distance slopes: 2^(-8 (h + 1) / H)


def _norm(name: str, d: int, eps: float) -> PartSpec:
    return PartSpec.make("rmsnorm", names={"weight": name}, size=d, eps=eps)


def _attention(p: str, d: int, m, eps: float) -> PartSpec:
    names = {"q_proj.weight": p + "q", "q_proj.bias": p + "q.b", "k_proj.weight": p + "k", "k_proj.bias": p + "k.b",
             "out_proj.weight": p + "o", "out_proj.bias": p + "o.b"}
    return PartSpec.make("attention", names=names, size=d, heads=m.heads, kv_heads=m.kv_heads, head_dim=m.dim,
                         qk_norm=False, norm_eps=eps, position=PartSpec.make("none"), window=m.window, scale=m.scale,
                         bias=True, values_are_keys=True, slope_exp=SLOPE_EXP,
                         q_temp=(m.q_temp_coef, m.q_temp_every) if m.q_temp_every else None)


def _retention(p: str, d: int, m, eps: float) -> PartSpec:
    names = {f"{t}.weight": p + t for t in ("q", "k", "v", "g", "o")}
    position = PartSpec.make("none")
    if m.rot_dims:
        position = PartSpec.make("rope", rot_dim=m.rot_dims, theta=m.rot_base, pairing="split_half", table64=True)
    return PartSpec.make("retention", names=names, size=d, heads=m.heads, key_dim=m.dim, value_dim=m.vdim,
                         decay=tuple(m.decay), norm_eps=eps, position=position)


def _feed_forward(p: str, d: int, f) -> PartSpec:
    if f.kind == "dense":
        return PartSpec.make("swiglu", names={"gate.weight": p + "gate", "up.weight": p + "up", "down.weight": p + "down"},
                             size=d, ff=f.ff)
    names = {"router.weight": p + "router"}
    for e in range(f.experts):
        names.update({f"e{e}.{t}.weight": f"{p}e{e}.{t}" for t in ("gate", "up", "down")})
    return PartSpec.make("moe", names=names, size=d, ff=f.ff, experts=f.experts, top=f.top, renormalize=False)


def build_spec(cfg: SamusunConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        mixer = (_attention if L.type == "attention" else _retention)(p + "mix.", d, L.mixer, eps)
        ffn = None if L.mlp is None else _feed_forward(p + "mlp.", d, L.mlp)
        layers.append(LayerSpec(norm1=_norm(p + "norm1", d, eps), mixer=mixer, norm2=None, ffn=ffn, arrangement="parallel"))
    schedule, connectors = None, []
    if cfg.loop is not None:
        lp = cfg.loop
        connectors = [PartSpec.make("add_step", names={"step": "loop.step"}, size=d, steps=lp.times)]
        schedule = [Run(i) for i in range(lp.start)]
        for t in range(lp.times):
            schedule += [Run(i, before=(0, t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        schedule += [Run(i) for i in range(lp.stop, len(cfg.layers))]
    return ModelSpec(architecture=NAME, hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
                     embedding=PartSpec.make("table", names={"weight": "embed"}, vocab=cfg.vocab, size=d,
                                             scale=cfg.embedding_scale),
                     layers=layers, final_norm=_norm("final.norm", d, eps),
                     head=PartSpec.make("linear", names={"weight": "head"}, vocab=cfg.vocab, size=d, tied=False,
                                        logit_scale=cfg.logit_scale, softcap=cfg.logit_softcap),
                     schedule=schedule or [], connectors=connectors)


register_architecture(NAME, SamusunConfig.from_dict, build_spec)
