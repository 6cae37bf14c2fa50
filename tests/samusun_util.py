"""Small Samusun configurations for the tests, their model folders (random weights in a temporary
folder), and helpers that run the engine and the plain implementation side by side.

The configurations differ from one another in every size: query heads equal to or a multiple of the key heads,
head sizes that are and are not multiples of 16, windows smaller and larger than a cache page (and of ONE
position, and longer than any prompt), rotary dimensions that cover the whole key or part of it or none, decays
near 1 and far from it, experts of which one, two or all are used, layers without a feed-forward, a loop over
the first, the last or all layers, and every order of layer kinds."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import numpy as np
import torch


def attention(heads, kv_heads, dim, window, scale, coef, every):
    return dict(dim=dim, heads=heads, kv_heads=kv_heads, mask=dict(size=window), q_temp=dict(coef=coef, every=every),
                scale=scale, vdim=dim)


def retention(heads, dim, vdim, decay, rot_dims, base):
    return dict(decay=list(decay), dim=dim, heads=heads, rot=dict(base=base, dims=rot_dims), vdim=vdim)


def dense(ff):
    return dict(ff=ff, kind="dense")


def moe(ff, experts, top):
    return dict(expert=dict(ff=ff), kind="moe", router=dict(experts=experts, top=top))


def layer(kind, mixer, mlp=None):
    return dict(type=kind, mixer=mixer, mlp=mlp)


def config(vocab, width, layers, loop=None, eps=1e-5, emb=0.7, logit_scale=1.3, cap=20.0):
    d = dict(architecture="Samusun", embedding=dict(scale=emb), layers=layers, logit_scale=logit_scale,
             logit_softcap=cap, norm=dict(eps=eps), vocab=vocab, width=width)
    if loop is not None:
        d["loop"] = dict(start=loop[0], stop=loop[1], times=loop[2])
    return d


# A: retention first, a loop of two passes over layers 1..2, window 21 (pages of 16 do not divide it), grouped keys,
# an attention layer without a feed-forward, five experts of which two are used
CFG_A = config(211, 96, [
    layer("retention", retention(3, 20, 12, [0.9, 0.99, 0.5], 8, 10000.0), moe(40, 5, 2)),
    layer("attention", attention(4, 2, 24, 21, 0.2, 0.25, 7), dense(160)),
    layer("attention", attention(6, 1, 16, 50, 0.31, 0.5, 3)),
], loop=(1, 3, 2))

# B: no loop; a window of ONE position and a window longer than any prompt; rotation over the whole key and none at
# all; one expert a token; three experts; keys of 40 (no multiple of 16: the kernels on CUDA cores in both dtypes)
CFG_B = config(300, 128, [
    layer("attention", attention(2, 2, 40, 1, 0.15, 0.1, 1), moe(24, 3, 1)),
    layer("retention", retention(2, 32, 48, [0.999, 0.75], 32, 500.0), dense(192)),
    layer("attention", attention(8, 4, 16, 4096, 0.25, 0.4, 64), moe(56, 4, 4)),
    layer("retention", retention(4, 8, 40, [1.0, 0.9, 0.8, 0.7], 0, 10000.0)),
], emb=1.0, logit_scale=0.8, cap=9.0)

# C: the loop is the whole model, three passes; one retention head of 64 x 64; a window equal to a page; every
# expert used
CFG_C = config(128, 64, [
    layer("attention", attention(2, 1, 32, 16, 0.18, 0.3, 5), moe(32, 2, 2)),
    layer("retention", retention(1, 64, 64, [0.97], 16, 1000000.0), dense(96)),
], loop=(0, 2, 3), eps=1e-6)

# D: sizes that are multiples of nothing: width 72, vocabulary 101, keys of 5 and 20, values of 7, a loop of one pass
# over the last layer, seven experts of 9
CFG_D = config(101, 72, [
    layer("retention", retention(3, 20, 7, [0.6, 0.95, 0.99], 6, 77.0), dense(40)),
    layer("attention", attention(3, 3, 5, 9, 0.45, 1.0, 2), moe(9, 7, 3)),
    layer("attention", attention(9, 3, 20, 33, 0.22, 0.05, 11), dense(24)),
], loop=(2, 3, 1))

# W: not tiny: the sizes at which the products run on their tensor-core kernels, the attention of portions on its
# own and the experts' grouped products on theirs
CFG_W = config(256, 1024, [
    layer("attention", attention(16, 4, 64, 100, 0.125, 0.35, 32), dense(2048)),
    layer("retention", retention(8, 128, 64, [1 - 2.0 ** -(3 + i) for i in range(8)], 64, 10000.0), moe(512, 8, 2)),
], emb=1.0, logit_scale=1.0)

CONFIGS = {"A": (CFG_A, 21), "B": (CFG_B, 22), "C": (CFG_C, 23), "D": (CFG_D, 24), "W": (CFG_W, 25)}
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_samusun_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from fellm_b200.weights import write_model_folder
    cfg, seed = CONFIGS[name]
    return str(write_model_folder(Path(_tmp.name) / f"samusun_{name}", cfg, seed))


def load_folder(folder):
    """(config dict, {name: float64 tensor}) read with the safetensors reader."""
    from fellm_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    w = {n: f.tensor(n).clone().double() for n in f.names()}
    f.close()
    return cfg, w


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return load_folder(model_folder(name))


def tokens(name: str, length: int, seed: int):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(3000 + seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=length)]


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int) -> torch.Tensor:
    import plain_samusun
    cfg, w = plain_model(name)
    return plain_samusun.forward(tokens(name, length, seed), w, cfg)


def make_engine(name_or_folder: str, dtype: str, **opts):
    from fellm_b200.config.options import EngineOptions
    from fellm_b200.engine import Engine
    folder = model_folder(name_or_folder) if name_or_folder in CONFIGS else name_or_folder
    o = dict(dtype=dtype, n_ctx=1024, ctx_past_model=True, max_requests=4, max_tokens=2048, page_tokens=16,
             cuda_graphs=False, n_batch=2048)
    o.update(opts)
    return Engine.open(folder, EngineOptions(**o))


def distance(got, want) -> float:
    """The largest, over the rows, root mean square difference of the logits with their means taken off,
    relative to the root mean square of the wanted logits."""
    got, want = got.double().cpu(), want.double().cpu()
    got = got - got.mean(-1, keepdim=True)
    want = want - want.mean(-1, keepdim=True)
    return float(((got - want).pow(2).mean(-1).sqrt() / want.pow(2).mean().sqrt()).max())


LIMIT = {"float32": 1e-4, "bfloat16": 6e-2}


def run_cuts(engine, req, toks, cuts):
    """Feeds toks in portions of the given sizes (the rest one by one) and returns the logits of every position."""
    from fellm_b200.engine import StepItem
    engine.add_request(req)
    out, at = [], 0
    sizes = list(cuts)
    while at < len(toks):
        n = sizes.pop(0) if sizes else 1
        n = min(n, len(toks) - at)
        out.append(engine.step([StepItem(req, toks[at:at + n], list(range(n)))]).clone())
        at += n
    engine.check_status()
    engine.release(req)
    return torch.cat(out)


def random_config(seed: int):
    """A configuration drawn at random: 2 to 5 layers of either kind in any order, heads and sizes that are and are
    not multiples of anything, windows from 1 to beyond the prompt, any feed-forward or none, a loop or none."""
    rng = np.random.default_rng(7000 + seed)
    pick = lambda xs: xs[int(rng.integers(0, len(xs)))]
    width = int(pick([48, 64, 72, 96, 128, 136]))
    n_layers = int(rng.integers(2, 6))
    layers = []
    for _ in range(n_layers):
        if rng.random() < 0.55:
            G = int(pick([1, 2, 3]))
            H = G * int(pick([1, 2, 4]))
            m = attention(H, G, int(pick([4, 8, 12, 16, 24, 32, 40, 48, 64])), int(pick([1, 2, 5, 15, 16, 17, 31, 40, 64, 100, 1000])),
                          float(rng.uniform(0.1, 0.5)), float(rng.uniform(0.0, 1.0)), int(pick([1, 2, 3, 7, 16, 50])))
            kind = "attention"
        else:
            H = int(pick([1, 2, 3, 5]))
            dk = int(pick([4, 8, 12, 16, 24, 32, 64, 96]))
            rot = int(pick([0, 2, dk // 2 - (dk // 2) % 2, dk]))
            m = retention(H, dk, int(pick([4, 8, 12, 20, 32, 64, 80])), [float(1.0 - 2.0 ** -rng.uniform(1, 9)) for _ in range(H)],
                          rot, float(pick([10.0, 10000.0, 1e6])))
            kind = "retention"
        r = rng.random()
        if r < 0.25:
            mlp = None
        elif r < 0.6:
            mlp = dense(int(pick([8, 24, 40, 64, 100, 160])))
        else:
            E = int(pick([1, 2, 3, 4, 6, 8, 12]))
            mlp = moe(int(pick([8, 9, 16, 24, 40, 64])), E, int(rng.integers(1, E + 1)))
        layers.append(layer(kind, m, mlp))
    loop = None
    if rng.random() < 0.6:
        a = int(rng.integers(0, n_layers))
        b = int(rng.integers(a + 1, n_layers + 1))
        loop = (a, b, int(rng.integers(1, 4)))
    return config(int(pick([50, 101, 128, 200, 333])), width, layers, loop=loop, eps=float(pick([1e-5, 1e-6])),
                  emb=float(rng.uniform(0.3, 2.0)), logit_scale=float(rng.uniform(0.3, 2.0)), cap=float(rng.uniform(5.0, 40.0)))
