"""Robazen: how the design is put together from parts.

A layer is `x += mixer(norm1(x))`, then `x += ff(norm2(x))` where the layer has a feed-forward; every
norm is Dynamic Tanh.  A layer's mixer is one of
  delta          gated delta rule, one decay per head, SiLU output gate           (parts/gated_delta.py)
  channel_delta  the same with a low-rank decay per key channel and a low-rank sigmoid gate
  parallel       two branches on the same input, each RMS-normed, averaged        (parts/parallel.py):
                 softmax attention inside blocks of positions, without rotation, soft-capped, gated per
                 head (parts/attention.py), and time mixing with a decaying state  (parts/timemix.py)
The feed-forward is W_down(SiLU(W_gate h) * W_up h).  `loop` repeats a run of layers with the same
weights, each pass with caches and states of its own; a pass opens with x <- W_in [x ; x0] + step[t]
(parts/connector.py).  Final norm, then the head.

Tensor names of the safetensors file: embed, head, final.norm{,.b,.alpha}, loop.in, loop.step, and per
layer i: l<i>.norm1{,.b,.alpha}, l<i>.norm2..., l<i>.mix.<tensor>, l<i>.mlp.{gate,up,down}.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.robazen import NAME, RobazenConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, Run

MAX_POSITION = 1 << 20        # the design has no learned or rotated positions: nothing ends a context but memory


def _norm(name: str, d: int) -> PartSpec:
    return PartSpec.make("dyt", names={"weight": name, "bias": name + ".b", "alpha": name + ".alpha"}, size=d)


def _delta(p: str, d: int, m, eps: float, channelwise: bool) -> PartSpec:
    names = {f"{t}.weight": p + t for t in ("q", "k", "v", "b", "o")}
    names.update({f"{t}.conv": f"{p}{t}.conv" for t in ("q", "k", "v")})
    names.update({"A_log": p + "A_log", "dt_bias": p + "dt_bias", "norm.weight": p + "norm"})
    if channelwise:
        names.update({f"{t}.weight": p + t for t in ("a1", "a2", "g1", "g2")})
    else:
        names.update({f"{t}.weight": p + t for t in ("a", "g")})
    return PartSpec.make("gated_delta", names=names, size=d, heads=m.heads, kv_heads=m.kv_heads, key_dim=m.dim,
                         value_dim=m.vdim, taps=m.conv, norm_eps=eps, decay="channel" if channelwise else "head",
                         gate="sigmoid_lowrank" if channelwise else "silu")


def _parallel(p: str, d: int, m, eps: float) -> PartSpec:
    L, R = m.left, m.right
    lp, rp = p + "left.", p + "right."
    left = PartSpec.make(
        "attention", names={"q_proj.weight": lp + "q", "k_proj.weight": lp + "k", "v_proj.weight": lp + "v",
                            "gate.weight": lp + "g", "out_proj.weight": lp + "o"},
        size=d, heads=L.heads, kv_heads=L.kv_heads, head_dim=L.dim, v_dim=L.vdim, qk_norm=False, norm_eps=eps,
        position=PartSpec.make("none"), window=None, scale=L.scale, softcap=L.softcap, chunk=L.chunk, head_gate=True)
    names = {f"{t}.weight": rp + t for t in ("r", "k", "v", "g", "w1", "w2", "o")}
    names.update({f"mu.{s}": f"{rp}mu.{s}" for s in ("r", "k", "v", "g", "w")})
    names.update({"w0": rp + "w0", "u": rp + "u", "norm.weight": rp + "norm"})
    right = PartSpec.make("time_mix", names=names, size=d, heads=R.heads, key_dim=R.dim, norm_eps=eps)
    return PartSpec.make("parallel", names={"out.0.weight": lp + "out", "out.1.weight": rp + "out"},
                         size=d, branches=(left, right), norm_eps=eps)


def build_spec(cfg: RobazenConfig) -> ModelSpec:
    d, eps = cfg.width, cfg.norm_eps
    layers = []
    for i, L in enumerate(cfg.layers):
        p = f"l{i}."
        if L.type == "parallel":
            mixer = _parallel(p + "mix.", d, L.mixer, eps)
        else:
            mixer = _delta(p + "mix.", d, L.mixer, eps, L.type == "channel_delta")
        ffn = None
        if L.ff is not None:
            ffn = PartSpec.make("swiglu", names={"gate.weight": p + "mlp.gate", "up.weight": p + "mlp.up",
                                                 "down.weight": p + "mlp.down"}, size=d, ff=L.ff)
        layers.append(LayerSpec(norm1=_norm(p + "norm1", d), mixer=mixer,
                                norm2=_norm(p + "norm2", d) if ffn is not None else None, ffn=ffn))
    schedule, connectors = None, []
    if cfg.loop is not None:
        lp = cfg.loop
        connectors = [PartSpec.make("concat_proj", names={"in.weight": "loop.in", "step": "loop.step"}, size=d,
                                    steps=lp.times)]
        schedule = [Run(i) for i in range(lp.start)]
        for t in range(lp.times):
            schedule += [Run(i, before=(0, t) if i == lp.start else None) for i in range(lp.start, lp.stop)]
        schedule += [Run(i) for i in range(lp.stop, len(cfg.layers))]
    return ModelSpec(architecture=NAME, hidden_size=d, vocab_size=cfg.vocab, max_position=MAX_POSITION,
                     embedding=PartSpec.make("table", names={"weight": "embed"}, vocab=cfg.vocab, size=d),
                     layers=layers, final_norm=_norm("final.norm", d),
                     head=PartSpec.make("linear", names={"weight": "head"}, vocab=cfg.vocab, size=d, tied=False),
                     schedule=schedule or [], connectors=connectors)


register_architecture(NAME, RobazenConfig.from_dict, build_spec)
