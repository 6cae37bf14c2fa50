"""Robazen on the GPU against the plain implementation (tests/plain_robazen.py).

First each mechanism alone, through its kernel's Python face with inputs made so that a fault shows
(one key that would win the softmax if a mask let it in, a write at token 0 read hundreds of tokens
later); then whole models of three configurations: whole prompts, prompts against token-by-token
decoding, portions down to two tokens, unequal batches against each request alone, pages and slots
that are freed and come again, long decoding, and greedy generation through the scheduler."""
from __future__ import annotations

import math

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import plain_robazen as P
import robazen_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


def _items(lengths):
    """item_start, item_slot for portions of these lengths in slots 2, 0, 3, ... (not the order of the items)."""
    starts = np.concatenate([[0], np.cumsum(lengths)])
    slots = [(2 + 3 * i) % 5 for i in range(len(lengths))]
    return _i32(starts), _i32(slots), slots


# ----------------------------------------------------------------------------- mechanisms alone

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_dyt_norm(dtype):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(0)
    x = torch.randn(37, 100, generator=g) * 3
    w, b = torch.rand(100, generator=g) + 0.5, torch.randn(100, generator=g)
    got = ops.dyt_norm(x.to(DEV), w.to(DEV), b.to(DEV), 0.7, dtype)
    want = P.dyt_norm(x.double(), w.double(), b.double(), 0.7)
    assert (got.double().cpu() - want).abs().max() < (1e-5 if dtype == torch.float32 else 3e-2)
    rows = _i32([5, 0, 36])
    got = ops.dyt_norm(x.to(DEV), w.to(DEV), b.to(DEV), 0.7, torch.float32, rows=rows)
    assert (got.double().cpu() - want[[5, 0, 36]]).abs().max() < 1e-5


@pytest.mark.parametrize("taps", [1, 2, 3, 4, 8])
def test_short_convolution_in_portions_equals_one_pass(taps):
    """Portions of 1, 2, 5, ... tokens through the state equal the convolution of the whole sequence, also where a
    portion is shorter than the history; two requests side by side in slots of their own."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(taps)
    C, T = 70, 241                                  # the last portion is longer than a block's tile of rows
    x = [torch.randn(T, C, generator=g) for _ in range(2)]
    w = torch.randn(C, taps, generator=g)
    want = [F.silu(P.causal_short_conv(xi.double(), w.double())) for xi in x]
    state = torch.zeros(5, max(taps - 1, 0), C, device=DEV)
    state[:] = 7.0                                  # other slots' contents must not matter
    cuts = [1, 2, 1, 5, 2, 9, 1, 20, 200]
    at = 0
    for n in cuts:
        starts, slots_t, slots = _items([n, n])
        if at == 0:
            for s in slots:
                state[s].zero_()
        rows = torch.cat([x[0][at:at + n], x[1][at:at + n]]).to(DEV)
        got = ops.causal_conv_act(rows, w.to(DEV), state, starts, slots_t, 2, n)
        for i in range(2):
            d = (got[i * n:(i + 1) * n].double().cpu() - want[i][at:at + n]).abs().max()
            assert d < 1e-5, (taps, at, n, i, float(d))
        at += n
    assert at == T


def test_token_shift_in_portions():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(3)
    d, T = 50, 223
    h = torch.randn(T, d, generator=g)
    mu = torch.rand(5, d, generator=g)
    prev = torch.cat([torch.zeros(1, d), h[:-1]])
    want = torch.stack([h + (prev - h) * mu[s] for s in range(5)])
    state = torch.zeros(4, d, device=DEV)
    at = 0
    for n in [1, 2, 7, 1, 12, 200]:
        got = ops.token_shift_mix(h[at:at + n].to(DEV).contiguous(), mu.to(DEV), state, _i32([0, n]), _i32([1]), 1, n)
        assert (got.cpu() - want[:, at:at + n]).abs().max() < 1e-6
        at += n


def test_lowrank_expand():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(4)
    T, R, H, per = 19, 24, 3, 10
    z = torch.randn(T, R + 6, generator=g)
    w2 = torch.randn(H * per, R, generator=g) * 0.3
    bias = torch.randn(H * per, generator=g)
    rate = torch.randn(H, generator=g)
    zz = z[:, 3:3 + R].double()
    lin = zz @ w2.double().T + bias.double()
    got = ops.lowrank_expand(z.to(DEV)[:, 3:3 + R], w2.to(DEV), bias.to(DEV))
    assert (got.double().cpu() - lin).abs().max() < 1e-5
    got = ops.lowrank_expand(z.to(DEV)[:, 3:3 + R], w2.to(DEV), bias.to(DEV), f_in="tanh", f_out="exp_neg_exp")
    want = torch.exp(-torch.exp(torch.tanh(zz) @ w2.double().T + bias.double()))
    assert (got.double().cpu() - want).abs().max() < 1e-6
    got = ops.lowrank_expand(z.to(DEV)[:, 3:3 + R], w2.to(DEV).bfloat16(), bias.to(DEV), f_out="decay_softplus",
                             rate=rate.to(DEV), per=per)
    lin_b = zz @ w2.bfloat16().double().T + bias.double()
    want = torch.exp(-torch.exp(rate.double()).repeat_interleave(per) * F.softplus(lin_b))
    assert (got.double().cpu() - want).abs().max() < 1e-6


def _delta_inputs(T, H, G, dk, dv, seed, channelwise):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(T, G, dk, generator=g)
    k = torch.randn(T, G, dk, generator=g)
    v = torch.randn(T, H, dv, generator=g)
    small = torch.randn(T, 2 * H + 3, generator=g)             # beta at 1 + h, the decay's logit at 1 + H + h
    A_log = torch.rand(H, generator=g) * 2 - 3
    dt_bias = torch.randn(H, generator=g)
    gch = torch.rand(T, H, dk, generator=g) * 0.2 + 0.8 if channelwise else None
    return q, k, v, small, A_log, dt_bias, gch


def _delta_want(q, k, v, small, A_log, dt_bias, gch):
    T, G, dk = q.shape
    H = v.shape[1]
    qd, kd = q.double(), k.double()
    qn = qd / torch.sqrt((qd * qd).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    kn = kd / torch.sqrt((kd * kd).sum(-1, keepdim=True) + 1e-6)
    beta = torch.sigmoid(small[:, 1:1 + H].double())
    if gch is None:
        dec = torch.exp(-torch.exp(A_log.double()) * F.softplus(small[:, 1 + H:1 + 2 * H].double() + dt_bias.double()))
    else:
        dec = gch.double()
    return P.delta_rule_scan(qn.repeat_interleave(H // G, 1), kn.repeat_interleave(H // G, 1), v.double(), beta, dec)


@pytest.mark.parametrize("H,G,dk,dv,channelwise", [(4, 2, 16, 24, False), (3, 3, 24, 16, True), (4, 1, 48, 40, True),
                                                   (2, 2, 8, 72, False), (2, 1, 128, 32, False), (1, 1, 200, 5, True)])
def test_delta_rule_scan(H, G, dk, dv, channelwise):
    """The scan in portions of 1, 2 and more tokens against the plain recurrence; key sizes on one lane, on several
    lanes and no power of two, value sizes that do not fill a warp."""
    from fellm_b200 import ops
    T = 45
    q, k, v, small, A_log, dt_bias, gch = _delta_inputs(T, H, G, dk, dv, 7, channelwise)
    want = _delta_want(q, k, v, small, A_log, dt_bias, gch).reshape(T, H * dv)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), torch.zeros(T, 5), v.reshape(T, -1)], 1).to(DEV)
    k_off, v_off = G * dk, 2 * G * dk + 5
    state = torch.full((3, H, dk, dv), 9.0, device=DEV)
    state[1].zero_()
    at = 0
    for n in [2, 1, 1, 17, 2, 22]:
        got = ops.delta_scan(qkv[at:at + n], k_off, v_off, small.to(DEV)[at:at + n], 1, 1 + H, A_log.to(DEV),
                             dt_bias.to(DEV), None if gch is None else gch[at:at + n].reshape(n, -1).contiguous().to(DEV),
                             state, _i32([0, n]), _i32([1]), 1, H, G, dk, dv)
        err = (got.double().cpu() - want[at:at + n]).abs().max()
        assert err < 2e-5, (at, n, float(err))
        at += n
    assert float(state[0].min()) == 9.0 and float(state[2].max()) == 9.0       # the neighbours' slots are untouched


def test_delta_rule_keeps_a_far_write():
    """With no decay and keys at right angles, what token 0 wrote is read back unchanged 600 tokens later."""
    from fellm_b200 import ops
    T, dk, dv = 601, 32, 16
    q = torch.zeros(T, 1, dk)
    k = torch.zeros(T, 1, dk)
    for t in range(T):
        k[t, 0, 1 + t % (dk - 1)] = 1.0                     # never channel 0 again
    k[0, 0] = 0
    k[0, 0, 0] = 1.0
    q[:, 0, 1] = 1.0
    q[T - 1, 0] = 0
    q[T - 1, 0, 0] = 1.0
    v = torch.randn(T, 1, dv, generator=torch.Generator().manual_seed(1))
    small = torch.zeros(T, 2)
    small[:, 0] = 30.0                                      # beta = 1
    small[:, 1] = -40.0                                     # softplus -> 0: decay 1
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(DEV)
    state = torch.zeros(1, 1, dk, dv, device=DEV)
    got = ops.delta_scan(qkv, dk, 2 * dk, small.to(DEV), 0, 1, torch.zeros(1, device=DEV), torch.zeros(1, device=DEV), None,
                         state, _i32([0, T]), _i32([0]), 1, 1, 1, dk, dv)
    assert (got[T - 1].cpu() - v[0, 0] * dk ** -0.5).abs().max() < 1e-5


@pytest.mark.parametrize("H,dk", [(3, 16), (1, 64), (4, 8), (2, 40), (1, 160)])
def test_decay_bonus_scan(H, dk):
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(H * 100 + dk)
    T = 33
    r, k, v = (torch.randn(T, H, dk, generator=g) for _ in range(3))
    w = torch.rand(T, H, dk, generator=g) * 0.5 + 0.5
    u = torch.randn(H, dk, generator=g)
    S = torch.zeros(H, dk, dk, dtype=torch.float64)
    want = torch.zeros(T, H, dk, dtype=torch.float64)
    for t in range(T):
        kv = torch.einsum("hk,hv->hkv", k[t].double(), v[t].double())
        want[t] = torch.einsum("hkv,hk->hv", S + u.double()[:, :, None] * kv, r[t].double())
        S = w[t].double()[:, :, None] * S + kv
    state = torch.zeros(2, H, dk, dk, device=DEV)
    at = 0
    for n in [1, 2, 9, 1, 20]:
        sl = slice(at, at + n)
        got = ops.decay_bonus_scan(r[sl].reshape(n, -1).to(DEV), k[sl].reshape(n, -1).to(DEV), v[sl].reshape(n, -1).to(DEV),
                                   w[sl].reshape(n, -1).to(DEV), u.to(DEV), state, _i32([0, n]), _i32([1]), 1, H, dk)
        err = (got.double().cpu() - want[sl].reshape(n, -1)).abs().max()
        assert err < 1e-4 * max(1.0, float(want.abs().max())), (at, n, float(err))
        at += n
    # (the kernel keeps a head's matrix column by column)
    assert (state[1].double().cpu().transpose(1, 2) - S).abs().max() < 1e-4 * max(1.0, float(S.abs().max()))


def test_head_norm_gate_and_branch_combine():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(5)
    T, H, dv = 9, 3, 20
    o = torch.randn(T, H * dv, generator=g)
    gate = torch.randn(T, H * dv, generator=g)
    for per_head, act in ((False, "silu"), (True, "sigmoid"), (True, None)):
        w = torch.rand(H * dv if per_head else dv, generator=g) + 0.5
        got = ops.head_norm_gate(o.to(DEV), w.to(DEV), per_head, gate.to(DEV) if act else None, act, 1e-5, H, dv, torch.float32)
        want = P.rms_unit(o.double().view(T, H, dv), 1e-5) * (w.double().view(H, dv) if per_head else w.double())
        want = want.reshape(T, -1) * (F.silu(gate.double()) if act == "silu" else torch.sigmoid(gate.double()) if act else 1.0)
        assert (got.double().cpu() - want).abs().max() < 1e-5
    d = 70
    x = torch.randn(T, d, generator=g)
    a, b = torch.randn(T, d, generator=g) * 3, torch.randn(T, d, generator=g) * 0.01
    wa, wb = torch.rand(d, generator=g), torch.rand(d, generator=g)
    xd = x.to(DEV).clone()
    ops.branch_combine(xd, [a.to(DEV), b.to(DEV)], [wa.to(DEV), wb.to(DEV)], 1e-5)
    want = x.double() + 0.5 * (P.rms_unit(a.double(), 1e-5) * wa.double() + P.rms_unit(b.double(), 1e-5) * wb.double())
    assert (xd.double().cpu() - want).abs().max() < 1e-5


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("chunk,page", [(24, 16), (7, 16), (80, 16), (64, 64), (16, 16)])
def test_attention_at_the_edges_of_chunks_and_pages(dtype, chunk, page):
    """Every query finds, at each earlier position, a key that would take all the weight if it were seen: the result
    must be the plain chunked attention, in which the key just outside the chunk does not count and the first key
    inside does.  Keys and values have different sizes; rows come as two requests whose pages interleave."""
    from fellm_b200 import ops
    H, G, hd, vd, T = 4, 2, 16, 24, 3 * max(chunk, page) + 5
    g = torch.Generator().manual_seed(chunk)
    W = {"q": torch.randn(H * hd, 32, generator=g), "k": torch.randn(G * hd, 32, generator=g) * 2,
         "v": torch.randn(G * vd, 32, generator=g), "g": torch.randn(H, 32, generator=g),
         "o": torch.eye(H * vd)}
    cfg = dict(heads=H, kv_heads=G, dim=hd, vdim=vd, scale=0.7, softcap=11.0, mask=dict(size=chunk))
    outs = []
    pool = torch.zeros(2 * (-(-T // page)) + 1, 1, G * page * (hd + vd), dtype=dtype, device=DEV)
    n_pages = -(-T // page)
    table = torch.full((2, n_pages), -1, dtype=torch.int32, device=DEV)
    for r in range(2):
        table[r] = torch.arange(n_pages, dtype=torch.int32) * 2 + (1 - r)          # the two requests' pages alternate
    hs = [torch.randn(T, 32, generator=g).to(dtype).float() for _ in range(2)]
    for r in range(2):
        h = hs[r]
        Wd = {n: t.to(dtype).float() for n, t in W.items()}
        want = P.chunked_attention(h.double(), {n: t.double() for n, t in Wd.items()}, "", cfg)
        qkv = (h @ torch.cat([Wd["q"], Wd["k"], Wd["v"]]).T).to(dtype).to(DEV)
        gate = (h @ Wd["g"].T).to(DEV)
        if dtype == torch.bfloat16:        # the oracle sees the rounded q, k, v the kernel sees
            q, k, v = qkv.float().cpu().split([H * hd, G * hd, G * vd], 1)
            Wi = {"q": torch.eye(H * hd), "k": torch.eye(G * hd), "v": torch.eye(G * vd)}
            want = _attention_from_qkv(q, k, v, gate.cpu(), cfg)
        got = []
        at = 0
        for n in [1, 2, page - 1, 1, chunk + 1, T]:          # portions that end before, on and behind the edges
            n = min(n, T - at)
            if n <= 0:
                break
            pos = _i32(list(range(at, at + n)))
            slot = _i32([r] * n)
            ops.kv_write(qkv[at:at + n], H * hd, (H + G) * hd, pool, table, pos, slot, 0, page, G, hd, vd)
            got.append(ops.paged_attention_general(qkv[at:at + n], H, hd, vd, pool, table, pos, slot, 0, page, G, 0.7,
                                                   chunk=chunk, softcap=11.0, gate=gate[at:at + n]))
            at += n
        got = torch.cat(got).double().cpu()
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max())), (r, float((got - want).abs().max()))


@pytest.mark.parametrize("hd,chunk,page,softcap", [(16, 24, 16, 9.0), (64, 100, 64, None), (48, 7, 16, 30.0), (32, 64, 32, 2.0)])
def test_tensor_core_attention_of_portions_with_cap_chunk_and_gate(hd, chunk, page, softcap):
    """The tensor-core kernel for portions (keys and values of one size) against the plain attention: three items of
    unequal length in one launch, each continuing a request at a position inside a chunk and inside a page."""
    from fellm_b200 import ops
    H, G = 6, 2
    g = torch.Generator().manual_seed(hd + chunk)
    cfg = dict(heads=H, kv_heads=G, dim=hd, vdim=hd, scale=0.4, mask=dict(size=chunk))
    if softcap:
        cfg["softcap"] = softcap
    lens, done = [70, 1, 33], [chunk + 3, 2 * page - 1, 0]                 # tokens of this step, tokens already in the cache
    n_pages = [-(-(a + b) // page) for a, b in zip(lens, done)]
    pool = torch.zeros(sum(n_pages) + 1, 2, 2, G, page, hd, dtype=torch.bfloat16, device=DEV)
    table = torch.full((3, max(n_pages)), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(sum(n_pages), generator=g).to(torch.int32)
    at = 0
    for r in range(3):
        table[r, :n_pages[r]] = perm[at:at + n_pages[r]]
        at += n_pages[r]
    rows, gates, wants, pos, slot, starts = [], [], [], [], [], [0]
    layer = 1
    for r in range(3):
        T = lens[r] + done[r]
        qkv = (torch.randn(T, (H + 2 * G) * hd + 8, generator=g) * 1.5).bfloat16()
        gate = torch.randn(T, H + 3, generator=g)
        q, k, v = qkv[:, :(H + 2 * G) * hd].float().split([H * hd, G * hd, G * hd], 1)
        wants.append(_attention_from_qkv(q, k, v, gate[:, :H], cfg)[done[r]:])
        dev = qkv.to(DEV)
        if done[r]:                     # what earlier steps left in the cache
            ops.kv_write(dev[:done[r]], H * hd, (H + G) * hd, pool, table, _i32(list(range(done[r]))), _i32([r] * done[r]),
                         layer, page, G, hd, hd)
        rows.append(dev[done[r]:])
        gates.append(gate[done[r]:])
        pos += list(range(done[r], T))
        slot += [r] * lens[r]
        starts.append(starts[-1] + lens[r])
    qkv_d, gate_d = torch.cat(rows).contiguous(), torch.cat(gates).to(DEV).contiguous()
    pos_d, slot_d = _i32(pos), _i32(slot)
    ops.kv_write(qkv_d, H * hd, (H + G) * hd, pool, table, pos_d, slot_d, layer, page, G, hd, hd)
    got = ops.attention_prefill_general(qkv_d, H, pool, table, pos_d, slot_d, _i32(starts), 3, max(lens), layer, 0.4,
                                        chunk=chunk, softcap=softcap, gate=gate_d).double().cpu()
    want = torch.cat(wants)
    assert (got - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max())), float((got - want).abs().max())
    # and the kernel on CUDA cores gives the same on the same cache
    simt = ops.paged_attention_general(qkv_d, H, hd, hd, pool, table, pos_d, slot_d, layer, page, G, 0.4, chunk=chunk,
                                       softcap=softcap, gate=gate_d).double().cpu()
    assert (simt - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max()))


def _attention_from_qkv(q, k, v, gate, cfg):
    H, G, hd, vd = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = q.shape[0]
    W = {"q": torch.eye(H * hd).double(), "k": torch.eye(G * hd).double(), "v": torch.eye(G * vd).double(),
         "o": torch.eye(H * vd).double()}
    # the plain function projects h itself: give it [q | k | v | gate] as h and selectors as weights
    h = torch.cat([q, k, v, gate], 1).double()
    n = h.shape[1]
    sel = lambda a, b: torch.eye(n, dtype=torch.float64)[a:b]
    Ws = {"q": sel(0, H * hd), "k": sel(H * hd, (H + G) * hd), "v": sel((H + G) * hd, (H + G) * hd + G * vd),
          "g": sel(n - H, n), "o": W["o"]}
    return P.chunked_attention(h, Ws, "", cfg)


# ----------------------------------------------------------------------------- whole models

@pytest.fixture(scope="module", params=["float32", "bfloat16"])
def engines(request):
    made = {}

    def get(name, **opts):
        key = (name, tuple(sorted(opts.items())))
        if key not in made:
            made[key] = U.make_engine(name, request.param, **opts)
        return made[key]
    get.dtype = request.param
    yield get
    made.clear()


@pytest.mark.parametrize("name", ["P", "Q", "R", "S"])
def test_whole_prompt(engines, name):
    T = 150
    eng = engines(name)
    got = U.run_cuts(eng, "a", U.tokens(name, T, 0), [T])
    d = U.distance(got, U.plain_logits(name, T, 0))
    assert d < U.LIMIT[engines.dtype], d


@pytest.mark.parametrize("name", ["P", "Q", "R"])
def test_layers_one_by_one(engines, name):
    """The residual stream after every layer run against the plain implementation's."""
    from fellm_b200.models import model as M
    cfg, w = U.plain_model(name)
    toks = U.tokens(name, 40, 1)
    _, want = P.forward(cfg, w, toks, keep_layers=True)
    kept, orig = [], M.Block.forward

    def fwd(self, x, *a, **k):
        r = orig(self, x, *a, **k)
        kept.append(x.clone())
        return r
    M.Block.forward = fwd
    try:
        U.run_cuts(engines(name), "a", toks, [40])
    finally:
        M.Block.forward = orig
    got = torch.stack(kept).double().cpu()
    assert got.shape == want.shape
    tol = 1e-4 if engines.dtype == "float32" else 6e-2
    for i in range(got.shape[0]):
        err = float((got[i] - want[i]).abs().max() / want[i].abs().max())
        assert err < tol, (i, err)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_prompt_against_token_by_token(engines, name):
    T = 90
    eng = engines(name)
    toks = U.tokens(name, T, 2)
    whole = U.run_cuts(eng, "a", toks, [T])
    single = U.run_cuts(eng, "b", toks, [])
    if engines.dtype == "float32":
        # every sum's order is set by the model's sizes, not by the cut: the 32-bit engine repeats itself bit for bit
        assert torch.equal(single, whole)
    assert U.distance(single, whole) < U.LIMIT["bfloat16"]
    assert U.distance(single, U.plain_logits(name, T, 2)) < U.LIMIT[engines.dtype]


@pytest.mark.parametrize("name,cuts", [("P", [2, 2, 3, 17, 2, 24, 1, 1, 23, 2, 48]), ("Q", [7, 2, 71, 2, 9, 80, 3]),
                                       ("R", [31, 2, 1, 32, 33, 2]), ("S", [8, 2, 9, 1, 10, 65])])
def test_portions_of_many_sizes(engines, name, cuts):
    T = 170
    eng = engines(name)
    toks = U.tokens(name, T, 3)
    got = U.run_cuts(eng, "a", toks, cuts)
    assert U.distance(got, U.plain_logits(name, T, 3)) < U.LIMIT[engines.dtype]


@pytest.mark.parametrize("name", ["P", "Q"])
def test_unequal_batch_against_each_alone_with_slots_and_pages_that_come_again(engines, name):
    """Four requests of different lengths share steps (portions beside single tokens), end at different times and
    are followed by new ones in the slots and pages they gave back; the pool holds less than all of them together."""
    from fellm_b200.engine import StepItem
    eng = engines(name, max_tokens=448)
    lengths = [97, 5, 140, 33, 61, 120, 2, 75]
    plans = {i: (U.tokens(name, n, 10 + i), [3, 1, 2, 40, 1, 1, 17, 2, 64][i % 3:]) for i, n in enumerate(lengths)}
    waiting, live, got = list(plans), {}, {i: [] for i in plans}
    step = 0
    while waiting or live:
        while waiting and len(live) < 4 and eng.cache.free_pages() * eng.cache.page_tokens >= lengths[waiting[0]] + 16 * len(live):
            i = waiting.pop(0)
            eng.add_request(i)
            live[i] = [0, list(plans[i][1])]
        items = []
        for i, st in live.items():
            if (step + i) % 5 == 4:
                continue                                    # left out of this step, goes on later
            n = min(st[1].pop(0) if st[1] else 1, len(plans[i][0]) - st[0])
            items.append((i, StepItem(i, plans[i][0][st[0]:st[0] + n], list(range(n)))))
            st[0] += n
        if items:
            lg = eng.step([it for _, it in items])
            at = 0
            for i, it in items:
                got[i].append(lg[at:at + len(it.tokens)].clone())
                at += len(it.tokens)
        for i in [i for i, st in live.items() if st[0] == len(plans[i][0])]:
            eng.release(i)
            del live[i]
        eng.cache.audit()
        step += 1
    eng.check_status()
    cfg, w = U.plain_model(name)
    for i in plans:
        want = P.forward(cfg, w, plans[i][0])
        d = U.distance(torch.cat(got[i]), want)
        assert d < U.LIMIT[engines.dtype], (i, d)


def test_wide_model(engines):
    """Width 1,024, heads of 64 and 128, pages of 64 tokens: the sizes at which the products run on their tensor-core
    kernels and the attention of portions on its own; portions, then token by token."""
    name, T = "W", 44
    toks = U.tokens(name, T, 7)
    got = U.run_cuts(engines(name, page_tokens=64), "a", toks, [30, 2, 5])
    assert U.distance(got, U.plain_logits(name, T, 7)) < U.LIMIT[engines.dtype]


def test_long_decoding(engines):
    name, T = "R", 420
    toks = U.tokens(name, T, 5)
    got = U.run_cuts(engines(name), "a", toks, [20])
    assert U.distance(got, U.plain_logits(name, T, 5)) < U.LIMIT[engines.dtype]


def test_scaled_queries_and_keys_show_a_wrong_mask(engines):
    """Attention weights and biases scaled so that a softmax is nearly one-hot: a key let in from outside its chunk, or
    a first key left out, would change the logits far beyond rounding.  Also a model whose chunk is ONE position."""
    import copy
    import json
    from pathlib import Path
    from fellm_b200.weights.safetensors_io import write_safetensors
    cfg = copy.deepcopy(U.CFG_P)
    cfg["layers"][0]["mixer"]["left"]["mask"]["size"] = 1 if engines.dtype == "float32" else 5
    cfg["layers"][0]["mixer"]["left"]["softcap"] = 200.0
    cfg["layers"][0]["mixer"]["left"]["scale"] = 1.0
    _, w = U.plain_model("P")
    w = {n: t.clone() for n, t in w.items()}
    for n in ("l0.mix.left.q", "l0.mix.left.k"):
        w[n] = (w[n].float() * 40).bfloat16()
    folder = Path(U._tmp.name) / f"sharp_{engines.dtype}"
    folder.mkdir(exist_ok=True)
    (folder / "config.json").write_text(json.dumps(cfg))
    write_safetensors(folder / "model.safetensors", w)
    eng = U.make_engine(str(folder), engines.dtype)
    toks = U.tokens("P", 64, 6)
    got = U.run_cuts(eng, "a", toks, [3, 2, 11, 1, 1, 30])
    want = P.forward(cfg, w, toks)
    assert U.distance(got, want) < U.LIMIT[engines.dtype]


@pytest.mark.parametrize("name", ["P", "Q"])
def test_greedy_generation_through_the_scheduler(name):
    """Engine.generate_batch (scheduler, sampler, CUDA graphs on) in float32 against the plain implementation's greedy
    continuation; prompts longer than a portion so that the scheduler cuts them."""
    from fellm_b200.engine import GenParams
    eng = U.make_engine(name, "float32", cuda_graphs=True, n_ubatch=32, n_batch=64, max_tokens=1024)
    cfg, w = U.plain_model(name)
    prompts = [U.tokens(name, n, 20 + i) for i, n in enumerate([70, 3, 41])]
    outs, stats = eng.generate_batch(prompts, GenParams.greedy(12))
    for p, got in zip(prompts, outs):
        seq = list(p)
        for k in range(12):
            lg = P.forward(cfg, w, seq)[-1]
            top = torch.topk(lg, 2).values
            if int(lg.argmax()) != got[k]:
                assert float(top[0] - top[1]) < 1e-4 * float(lg.abs().max()), (k, got, int(lg.argmax()))
                break
            seq.append(got[k])
    assert all(s is not None for s in stats)


def test_command_line_runs_the_design(capsys):
    from fellm_b200 import cli
    folder = U.model_folder("P")
    assert cli.main(["inspect", "--model", folder]) == 0
    out = capsys.readouterr().out
    assert "architecture: Robazen" in out and "l0.mix.left.q" in out
    assert cli.main(["run", folder, "--prompt", "5 17 3 9 100", "--max-tokens", "6", "--temperature", "0", "--dtype", "float32",
                     "--page-tokens", "16", "-c", "256", "--kv-device-budget", "4194304"]) == 0
    toks = [int(t) for t in capsys.readouterr().out.split()]
    cfg, w = U.plain_model("P")
    seq = [5, 17, 3, 9, 100]
    for t in toks:
        lg = P.forward(cfg, w, seq)[-1]
        top = torch.topk(lg, 2).values
        assert int(lg.argmax()) == t or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
        seq.append(t)
    assert len(toks) == 6


def test_bfloat16_generation_runs_through_the_entry_point():
    from fellm_b200.engine import GenParams
    eng = U.make_engine("R", "bfloat16", cuda_graphs=True, n_ubatch=16, n_batch=64)
    out = list(eng.generate(U.tokens("R", 50, 30), GenParams.greedy(20)))
    assert len(out) == 20 and all(0 <= t < U.CFG_R["vocab"] for t in out)
