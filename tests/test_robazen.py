"""Robazen without a GPU: the configuration reader, the model description made from it, the tensors it
asks for, what its layers keep between steps, and the plain implementation's own mechanisms."""
from __future__ import annotations

import copy

import pytest
import torch

import plain_robazen as P
import robazen_util as U
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
        assert arch.name == "Robazen" and c.to_dict() == cfg, name
        assert spec.vocab_size == cfg["vocab"] and spec.hidden_size == cfg["width"]
    # `architectures` (a list) names the design as well as `architecture`
    cfg = copy.deepcopy(U.CFG_Q)
    cfg["architectures"] = [cfg.pop("architecture")]
    assert _spec(cfg)[0].name == "Robazen"


@pytest.mark.parametrize("path,value,word", [
    (("width",), None, "width"), (("norm",), {}, "norm.eps"), (("layers", 0, "type"), "conv", "layers[0].type"),
    (("layers", 1, "mixer", "heads"), 3, "kv_heads"), (("layers", 0, "mixer", "left", "mask"), {}, "mask.size"),
    (("layers", 0, "mlp", "kind"), "routed", "mlp.kind"), (("loop", "stop"), 9, "loop"),
    (("layers", 0, "mixer", "left", "softcap"), -1.0, "softcap"), (("layers", 2, "mixer", "conv"), "3", "conv")])
def test_config_errors_name_the_key(path, value, word):
    cfg = copy.deepcopy(U.CFG_P)
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
    _, _, spec = _spec(U.CFG_P)                      # layers 0, 1 three times, then 2
    assert [(r.layer, r.before) for r in spec.schedule] == [
        (0, (0, 0)), (1, None), (0, (0, 1)), (1, None), (0, (0, 2)), (1, None), (2, None)]
    assert [i for i, _, _ in P.layer_order(U.CFG_P)] == [r.layer for r in spec.schedule]
    _, _, spec = _spec(U.CFG_Q)
    assert [(r.layer, r.before) for r in spec.schedule] == [(i, None) for i in range(4)] and not spec.connectors


def test_tensor_names_and_ranks_from_the_file():
    _, _, spec = _spec(U.CFG_Q)
    model = build_model(spec, "float32")
    table = model.param_table()
    for n in ("embed", "head", "final.norm", "final.norm.b", "final.norm.alpha", "l0.mix.a1", "l0.mix.g2", "l0.mix.q.conv",
              "l1.mix.left.g", "l1.mix.left.out", "l1.mix.right.mu.w", "l1.mix.right.w2", "l1.mix.right.u", "l2.mix.a",
              "l2.mix.dt_bias", "l2.mlp.down", "l2.norm2.alpha", "l3.mix.right.out"):
        assert n in table, n
    assert "l1.norm2" not in table and "loop.in" not in table            # no feed-forward there, no loop
    # the rank of a low-rank projection is whatever the file has, as long as its two factors agree
    decl = table["l0.mix.a1"][2]
    assert decl.fits((5, 128)) and decl.fits((31, 128)) and not decl.fits((5, 64))
    assert table["l0.mix.a2"][2].fits((4 * 48, 5))


def test_cache_needs_and_chunk_trimming():
    _, _, spec = _spec(U.CFG_P)
    needs = build_model(spec, "float32").cache_needs()
    par = needs[0]
    assert par[0] == PagedKV(2, 16, None, 24, 24) and par[1] == FixedState((96,)) and par[2] == FixedState((3, 16, 16))
    assert needs[1] == [FixedState((3, 2 * 2 * 16 + 4 * 24)), FixedState((4, 16, 24))]
    # a chunked layer gives back the pages in front of the chunk the next position lies in
    cm = CacheManager([PagedKV(1, 8, None, 24, None)], page_tokens=16, max_tokens=64, max_requests=2, n_ctx=512,
                      dtype=torch.float32, device="cpu")
    cm.add_request("a")
    held = []
    for _ in range(200):
        cm.reserve("a", 1)
        cm.advance("a", 1)
        cm.audit()
        held.append(4 - cm.free_pages())
        start = (cm.length("a") // 24) * 24
        first = cm.paged[0].first_page[0]
        assert first == start // 16                          # nothing the next query can see was given back
    assert max(held) <= 3                                    # 200 positions went through a pool of 64


def test_plain_mechanisms():
    torch.manual_seed(0)
    # a convolution whose last tap is 1 and the others 0 is the identity; zeros stand before the start
    x = torch.randn(6, 3, dtype=torch.float64)
    taps = torch.zeros(3, 4, dtype=torch.float64)
    taps[:, -1] = 1
    assert torch.equal(P.causal_short_conv(x, taps), x)
    taps[:, -1], taps[:, 0] = 0, 1
    assert torch.equal(P.causal_short_conv(x, taps)[3:], x[:3]) and float(P.causal_short_conv(x, taps)[:3].abs().max()) == 0
    # delta rule with beta = 1, no decay: a key's value is replaced, not added to
    k = torch.zeros(3, 1, 4, dtype=torch.float64)
    k[:, 0, 2] = 1
    v = torch.randn(3, 1, 5, dtype=torch.float64)
    o = P.delta_rule_scan(k, k, v, torch.ones(3, 1, dtype=torch.float64), torch.ones(3, 1, dtype=torch.float64))
    assert torch.allclose(o, v)
    # chunked attention: position i of a chunk of 3 averages v over the chunk's positions up to i when q = 0
    W = {"q": torch.zeros(2, 2, dtype=torch.float64), "k": torch.eye(2, dtype=torch.float64),
         "v": torch.eye(2, dtype=torch.float64), "g": torch.zeros(1, 2, dtype=torch.float64), "o": torch.eye(2, dtype=torch.float64)}
    h = torch.randn(7, 2, dtype=torch.float64)
    cfg = dict(heads=1, kv_heads=1, dim=2, vdim=2, scale=1.0, softcap=3.0, mask=dict(size=3))
    a = P.chunked_attention(h, W, "", cfg)
    assert torch.allclose(a[4], 0.5 * h[3:5].mean(0)) and torch.allclose(a[3], 0.5 * h[3]) and torch.allclose(a[2], 0.5 * h[:3].mean(0))


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_written_folder_is_read_back_and_runs_in_the_plain_implementation(name):
    cfg, w = U.plain_model(name)
    assert cfg == U.CONFIGS[name][0]
    assert w["final.norm.alpha"].shape == () and w["embed"].dtype == torch.bfloat16
    lg = U.plain_logits(name, 12, 0)
    assert lg.shape == (12, cfg["vocab"]) and bool(torch.isfinite(lg).all())
    # every position depends on the ones before it only
    lg2 = P.forward(cfg, w, U.tokens(name, 12, 0)[:7])
    assert torch.allclose(lg[:7], lg2, atol=1e-9)
