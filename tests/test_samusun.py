"""Samusun without a GPU: the configuration reader, the model description made from it, the tensors it
asks for, what its layers keep between steps, and the plain implementation's own mechanisms."""
from __future__ import annotations

import copy
import math

import pytest
import torch

import plain_samusun as P
import samusun_util as U
from fellm_b200.cache.manager import CacheManager
from fellm_b200.config.errors import ConfigError
from fellm_b200.config.registry import config_from_dict
from fellm_b200.models.model import build_model
from fellm_b200.parts.base import FixedState, PagedKV


def _spec(cfg):
    arch, c = config_from_dict(cfg)
    return arch, c, arch.build_spec(c)


def test_config_round_trip_and_registry():
    for name, (cfg, _) in U.CONFIGS.items():
        arch, c, spec = _spec(cfg)
        assert arch.name == "Samusun" and c.to_dict() == cfg, name
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"]
        assert all(ls.arrangement == "parallel" and ls.norm2 is None for ls in spec.layers)


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("norm",), {}, "norm.eps"), (("layers", 0, "type"), "conv", "layers[0].type"),
    (("layers", 1, "mixer", "heads"), 3, "kv_heads"), (("layers", 1, "mixer", "mask"), {}, "mask.size"),
    (("layers", 1, "mixer", "vdim"), 8, "vdim"), (("layers", 1, "mixer", "q_temp", "every"), 0, "q_temp.every"),
    (("layers", 0, "mixer", "decay"), [0.5], "decay"), (("layers", 0, "mixer", "rot", "dims"), 7, "rot.dims"),
    (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"), (("layers", 0, "mlp", "router", "top"), 6, "router.top"),
    (("layers", 0, "mlp", "expert"), {}, "expert.ff"), (("loop", "stop"), 9, "loop"), (("logit_softcap",), -2.0, "logit_softcap")])
def test_config_errors_name_the_key(path, value, word):
    cfg = copy.deepcopy(U.CFG_A)
    d = cfg
    for k in path[:-1]:
        d = d[k]
    if value is None:
        del d[path[-1]]
    else:
        d[path[-1]] = value
    with pytest.raises(ConfigError) as e:
        _spec(cfg)
    assert word in str(e.value)


def test_schedule_of_a_loop():
    _, _, spec = _spec(U.CFG_A)                      # layer 0, then layers 1, 2 twice
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, None), (1, (0, 0)), (2, None), (1, (0, 1)), (2, None)]
    assert [i for i, _ in P.layer_order(U.CFG_A)] == [r.layer for r in spec.schedule]
    _, _, spec = _spec(U.CFG_B)
    assert [(r.layer, r.before) for r in spec.schedule] == [(i, None) for i in range(4)] and not spec.connectors
    _, _, spec = _spec(U.CFG_C)
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, (0, 0)), (1, None), (0, (0, 1)), (1, None), (0, (0, 2)), (1, None)]
    _, _, spec = _spec(U.CFG_D)                      # one pass is still a pass: its step vector is added
    assert [(r.layer, r.before) for r in spec.schedule] == [(0, None), (1, None), (2, (0, 0))]


def test_tensor_names():
    _, _, spec = _spec(U.CFG_A)
    table = build_model(spec, "float32").param_table()
    for n in ("embed", "head", "final.norm", "loop.step", "l0.norm1", "l0.mix.q", "l0.mix.g", "l0.mix.o", "l0.mlp.router",
              "l0.mlp.e0.gate", "l0.mlp.e4.down", "l1.mix.q", "l1.mix.q.b", "l1.mix.k.b", "l1.mix.o.b", "l1.mlp.gate",
              "l2.mix.k"):
        assert n in table, n
    for n in ("l1.mix.v", "l1.norm2", "l2.mlp.gate", "l0.mlp.e5.gate", "l0.mix.q.b", "loop.in"):
        assert n not in table, n
    assert table["loop.step"][2].shape == (2, 96) and table["l1.mix.k"][2].shape == (2 * 24, 96)
    assert table["l0.mlp.e1.down"][2].shape == (96, 40) and table["l0.mlp.router"][2].shape == (5, 96)
    _, _, spec = _spec(U.CFG_B)
    assert "loop.step" not in build_model(spec, "float32").param_table()


def test_cache_needs_and_window_trimming():
    _, _, spec = _spec(U.CFG_A)
    needs = build_model(spec, "float32").cache_needs()
    assert needs[0] == FixedState((3, 20, 12))
    assert needs[1] == PagedKV(2, 24, 21, None, None, True) and needs[1].value_dim == 0      # the keys alone are kept
    assert needs[2] == PagedKV(1, 16, 50, None, None, True)
    assert needs[3] == needs[1] and needs[4] == needs[2]                                      # each pass has its own
    # the keys of a window: a request of any length holds window / page + 2 pages at most
    cm = CacheManager([PagedKV(1, 8, 21, None, None, True)], page_tokens=16, max_tokens=64, max_requests=2, n_ctx=512,
                      dtype=torch.float32, device="cpu")
    assert cm.paged[0].pool.shape[-1] == 1 * 16 * 8
    cm.add_request("a")
    for _ in range(200):
        cm.reserve("a", 1)
        cm.advance("a", 1)
        cm.audit()
        first = cm.paged[0].first_page[0]
        assert first * 16 <= max(0, cm.length("a") - 21 + 1)          # nothing the next query can see was given back
        assert 4 - cm.free_pages() <= 3


def test_plain_mechanisms():
    torch.manual_seed(0)
    f64 = torch.float64
    # query temperature: 1 until position every - 1, then 1 + coef ln 2, ...
    qt = P.query_temperature(10, 0.5, 4, f64)
    assert float(qt[2]) == 1.0 and abs(float(qt[3]) - (1 + 0.5 * math.log(2))) < 1e-12 and abs(float(qt[7]) - (1 + 0.5 * math.log(3))) < 1e-12
    assert abs(float(P.distance_slopes(4, f64)[1]) - 2.0 ** -4) < 1e-15 and abs(float(P.distance_slopes(4, f64)[3]) - 2.0 ** -8) < 1e-15
    # attention with q = 0 and no slope: the mean of the last `window` values, which are the keys
    k = torch.randn(9, 1, 3, dtype=f64)
    o = P.windowed_attention(torch.zeros(9, 2, 3, dtype=f64), k, k, 1.0, 4, torch.zeros(2, dtype=f64))
    assert torch.allclose(o[6, 1], k[3:7, 0].mean(0)) and torch.allclose(o[2, 0], k[:3, 0].mean(0))
    # a steep slope leaves the query's own position
    o = P.windowed_attention(torch.zeros(9, 2, 3, dtype=f64), k, k, 1.0, 4, torch.full((2,), 1e3, dtype=f64))
    assert torch.allclose(o[6, 0], k[6, 0])
    # rotation: position 0 is left alone; an angle of pi / 2 turns (u, v) into (-v, u); elements behind `dims` pass
    x = torch.randn(2, 1, 6, dtype=f64)
    r = P.rotate_half_partial(x, 4, 1.0)                       # both frequencies 1: angle = position
    assert torch.equal(r[0], x[0]) and torch.equal(r[:, :, 4:], x[:, :, 4:])
    assert torch.allclose(r[1, 0, 0], x[1, 0, 0] * math.cos(1) - x[1, 0, 2] * math.sin(1))
    assert torch.allclose(r[1, 0, 3], x[1, 0, 3] * math.cos(1) + x[1, 0, 1] * math.sin(1))
    # retention with decay 1 and q = k = e_0: the running sum of v; with decay 1/2 the halved sum
    q = torch.zeros(4, 1, 3, dtype=f64)
    q[:, 0, 0] = 1
    v = torch.randn(4, 1, 2, dtype=f64)
    assert torch.allclose(P.retention_scan(q, q, v, torch.ones(1, dtype=f64))[:, 0], v[:, 0].cumsum(0))
    o = P.retention_scan(q, q, v, torch.full((1,), 0.5, dtype=f64))
    assert torch.allclose(o[2, 0], v[2, 0] + 0.5 * v[1, 0] + 0.25 * v[0, 0])
    # routed experts: with one expert of E chosen the result is that expert's, weighted by its softmax score
    d, E = 4, 3
    W = {"router": torch.randn(E, d, dtype=f64)}
    for e in range(E):
        W.update({f"e{e}.gate": torch.randn(5, d, dtype=f64), f"e{e}.up": torch.randn(5, d, dtype=f64), f"e{e}.down": torch.randn(d, 5, dtype=f64)})
    h = torch.randn(6, d, dtype=f64)
    out = P.routed_experts(h, W, "", dict(experts=E, top=1))
    s = torch.softmax(h @ W["router"].T, -1)
    for t in range(6):
        e = int(s[t].argmax())
        assert torch.allclose(out[t], s[t, e] * P.gated_ff(h[t:t + 1], W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"])[0])
    # all experts chosen: the weights sum to 1
    out = P.routed_experts(h, W, "", dict(experts=E, top=E))
    want = sum(s[:, e:e + 1] * P.gated_ff(h, W[f"e{e}.gate"], W[f"e{e}.up"], W[f"e{e}.down"]) for e in range(E))
    assert torch.allclose(out, want)


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_written_folder_is_read_back_and_runs_in_the_plain_implementation(name):
    cfg, w = U.plain_model(name)
    assert cfg == U.CONFIGS[name][0]
    lg = U.plain_logits(name, 12, 0)
    assert lg.shape == (12, cfg["vocab"]) and bool(torch.isfinite(lg).all())
    assert float(lg.abs().max()) < cfg["logit_softcap"]
    # every position depends on the ones before it only
    lg2 = P.forward(U.tokens(name, 12, 0)[:7], w, cfg)
    assert torch.allclose(lg[:7], lg2, atol=1e-9)
