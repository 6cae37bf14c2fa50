"""Small Robazen configurations for the tests, their model folders (random weights in a temporary
folder), and helpers that run the engine and the plain implementation side by side.

The configurations differ from one another in every size: heads equal to or a multiple of the key
heads, key and value sizes that are equal or not, chunks that are no power of two and smaller or
larger than a cache page, 2 to 4 convolution taps, ranks, a loop of two or three passes or none,
feed-forwards on any kind of layer, and every order of layer kinds."""
from __future__ import annotations

import functools
import json
import tempfile
from pathlib import Path

import numpy as np
import torch


def delta(heads, kv_heads, dim, vdim, conv):
    return dict(conv=conv, dim=dim, heads=heads, kv_heads=kv_heads, vdim=vdim)


def parallel(heads, kv_heads, dim, vdim, chunk, scale, softcap, r_heads, r_dim):
    left = dict(dim=dim, heads=heads, kv_heads=kv_heads, mask=dict(size=chunk), scale=scale, vdim=vdim)
    if softcap is not None:
        left["softcap"] = softcap
    return dict(left=left, right=dict(dim=r_dim, heads=r_heads))


def layer(kind, mixer, ff=None):
    return dict(type=kind, mixer=mixer, mlp=None if ff is None else dict(ff=ff, kind="dense"))


# P: parallel first, a loop of three passes over two layers, chunk 24 (pages of 16 do not divide it)
CFG_P = dict(architecture="Robazen", vocab=211, width=96, norm=dict(eps=1e-5), layers=[
    layer("parallel", parallel(4, 2, 16, 24, 24, 0.25, 5.0, 3, 16), ff=160),
    layer("delta", delta(4, 2, 16, 24, 4)),
    layer("channel_delta", delta(3, 3, 24, 16, 2), ff=128),
], loop=dict(start=0, stop=2, times=3))

# Q: no loop, key size 48 (two lanes a column), value size 40 (no multiple of 32), chunk 80 > page, no soft cap,
# one key head for all heads, a single-head time mix
CFG_Q = dict(architecture="Robazen", vocab=300, width=128, norm=dict(eps=1e-6), layers=[
    layer("channel_delta", delta(4, 1, 48, 40, 3)),
    layer("parallel", parallel(6, 1, 32, 32, 80, 0.2, None, 1, 64), ff=None),
    layer("delta", delta(2, 2, 8, 72, 2), ff=192),
    layer("parallel", parallel(2, 2, 48, 16, 7, 0.3, 30.0, 4, 8), ff=64),
])

# R: a loop that is the whole model, run twice; key size 128
CFG_R = dict(architecture="Robazen", vocab=128, width=64, norm=dict(eps=1e-5), layers=[
    layer("delta", delta(2, 1, 128, 32, 3), ff=96),
    layer("parallel", parallel(2, 1, 64, 96, 32, 0.15, 40.0, 2, 32), ff=96),
], loop=dict(start=0, stop=2, times=2))

# S: sizes that are multiples of nothing: key sizes 5 and 20, value sizes 7 and 12, three heads, 15 time-mix channels,
# a vocabulary of 101, one convolution tap, a loop of one pass over the last layer
CFG_S = dict(architecture="Robazen", vocab=101, width=72, norm=dict(eps=1e-5), layers=[
    layer("delta", delta(3, 3, 5, 7, 1), ff=40),
    layer("parallel", parallel(3, 1, 20, 12, 9, 0.22, 15.0, 3, 5), ff=None),
    layer("channel_delta", delta(6, 2, 10, 3, 5), ff=24),
], loop=dict(start=2, stop=3, times=1))

# W: not tiny in width: the sizes at which a decode step's products take the norm in, and the attention of portions
# runs on tensor cores (keys and values of one size)
CFG_W = dict(architecture="Robazen", vocab=256, width=1024, norm=dict(eps=1e-5), layers=[
    layer("delta", delta(8, 4, 64, 128, 4), ff=2048),
    layer("parallel", parallel(16, 8, 64, 64, 32, 0.11, 30.0, 16, 64), ff=2048),
])

CONFIGS = {"P": (CFG_P, 11), "Q": (CFG_Q, 12), "R": (CFG_R, 13), "S": (CFG_S, 14), "W": (CFG_W, 15)}
_tmp = tempfile.TemporaryDirectory(prefix="fellm_b200_robazen_")


@functools.lru_cache(maxsize=None)
def model_folder(name: str) -> str:
    from fellm_b200.weights import write_model_folder
    cfg, seed = CONFIGS[name]
    return str(write_model_folder(Path(_tmp.name) / f"robazen_{name}", cfg, seed))


def load_folder(folder):
    """(config dict, {name: float tensor}) read with the safetensors reader."""
    from fellm_b200.weights.safetensors_io import SafetensorsFile
    cfg = json.loads((Path(folder) / "config.json").read_text())
    f = SafetensorsFile(Path(folder) / "model.safetensors")
    w = {n: f.tensor(n).clone() for n in f.names()}
    f.close()
    return cfg, w


@functools.lru_cache(maxsize=None)
def plain_model(name: str):
    return load_folder(model_folder(name))


def tokens(name: str, length: int, seed: int):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(2000 + seed)
    return [int(t) for t in rng.integers(0, cfg["vocab"], size=length)]


@functools.lru_cache(maxsize=None)
def plain_logits(name: str, length: int, seed: int) -> torch.Tensor:
    import plain_robazen
    cfg, w = plain_model(name)
    return plain_robazen.forward(cfg, w, tokens(name, length, seed))


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


def run_cuts(engine, req, toks, cuts, want_all=True):
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
