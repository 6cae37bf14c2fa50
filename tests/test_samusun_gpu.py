"""Samusun on the GPU against the plain implementation (tests/plain_samusun.py).

First each mechanism alone, through its kernel's Python face with inputs made so that a fault shows (one key that
would win the softmax if the window let it in, a write at token 0 read hundreds of tokens later, experts whose
outputs differ by orders of magnitude); then whole models of four configurations: whole prompts, layer by layer,
prompts against token-by-token decoding, portions down to two tokens, unequal batches against each request alone,
pages and slots that are freed and come again, long decoding past every window, and greedy generation through the
scheduler and the command line."""
from __future__ import annotations

import copy
import json
import math
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.nn.functional as F

import plain_samusun as P
import samusun_util as U

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _i32(xs):
    return torch.tensor(xs, dtype=torch.int32, device=DEV)


# ----------------------------------------------------------------------------- mechanisms alone

def test_embedding_scale_step_vector_and_capped_logits():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(1)
    table = torch.randn(50, 24, generator=g).bfloat16()
    toks = [3, 49, 0, 7]
    out = torch.empty(4, 24, device=DEV)
    ops.embed_rows(_i32(toks), table.to(DEV), out, None, 0.37)
    assert torch.equal(out.cpu(), table[toks].float() * 0.37)
    v = torch.randn(24, generator=g)
    x = out.clone()
    ops.add_row_vector(x, v.to(DEV))
    assert torch.equal(x.cpu(), out.cpu() + v)
    z = torch.randn(5, 33, generator=g) * 40
    got = ops.scale_softcap(z.to(DEV).clone(), 0.5, 15.0)
    assert (got.cpu().double() - 15.0 * torch.tanh(z.double() * 0.5 / 15.0)).abs().max() < 1e-5
    assert torch.equal(ops.scale_softcap(z.to(DEV).clone(), 2.0, None).cpu(), z * 2.0)


def test_unit_norm_of_heads_without_a_weight():
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(2)
    T, H, dv = 7, 3, 20
    o, gate = torch.randn(T, H * dv, generator=g) * 5, torch.randn(T, H * dv + 4, generator=g)
    got = ops.head_norm_gate(o.to(DEV), None, False, gate.to(DEV)[:, 4:], "silu", 1e-5, H, dv, torch.float32)
    want = P.rms_unit(o.double().view(T, H, dv), 1e-5).reshape(T, -1) * F.silu(gate[:, 4:].double())
    assert (got.double().cpu() - want).abs().max() < 1e-5


def _windowed_want(q, k, cfg, positions0=0):
    """The plain attention on q [T, H*hd], k [T, G*hd] as the kernel sees them (values = keys)."""
    T = q.shape[0]
    H, G, hd = cfg["heads"], cfg["kv_heads"], cfg["dim"]
    qt = P.query_temperature(T, cfg["q_temp"]["coef"], cfg["q_temp"]["every"], torch.float64)
    qq = q.double().view(T, H, hd) * qt[:, None, None]
    kk = k.double().view(T, G, hd)
    return P.windowed_attention(qq, kk, kk, cfg["scale"], cfg["mask"]["size"], P.distance_slopes(H, torch.float64)).reshape(T, -1)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("window,page,hd", [(21, 16, 24), (1, 16, 8), (16, 16, 40), (17, 16, 16), (64, 64, 16), (200, 16, 5), (33, 32, 48)])
def test_attention_at_the_edges_of_windows_and_pages(dtype, window, page, hd):
    """Keys are large and nearly alike in direction, so the softmax is sharp and dominated by whichever old key is
    seen: the key just outside the window must not count and the oldest inside must; the slopes and the query
    temperature (a step every 3 positions) move the winner.  The values are the keys: the cache holds keys alone.
    Rows come as two requests whose pages interleave, in portions that end before, on and behind the edges, single
    rows among them; one to four warps share a row's keys."""
    from fellm_b200 import ops
    H, G, T = 4, 2, 2 * max(window, page) + 7
    T = min(T, 150)
    cfg = dict(heads=H, kv_heads=G, dim=hd, scale=0.6, mask=dict(size=window), q_temp=dict(coef=0.8, every=3))
    g = torch.Generator().manual_seed(window * 7 + hd)
    n_pages = -(-T // page)
    pool = torch.zeros(2 * n_pages + 1, 1, G * page * hd, dtype=dtype, device=DEV)
    table = torch.full((2, n_pages), -1, dtype=torch.int32, device=DEV)
    for r in range(2):
        table[r] = torch.arange(n_pages, dtype=torch.int32) * 2 + (1 - r)
    slopes = P.distance_slopes(H, torch.float64).float().to(DEV)
    for r in range(2):
        q = (torch.randn(T, H * hd, generator=g) * 1.5).to(dtype).float()
        k = (torch.randn(T, G * hd, generator=g) * 2.0).to(dtype).float()
        want = _windowed_want(q, k, cfg)
        qk = torch.cat([q, torch.zeros(T, 3), k, torch.zeros(T, 2)], 1).to(dtype).to(DEV)     # q at 0, k at an odd column
        k_off = H * hd + 3
        got, at = [], 0
        for n in [1, 2, page - 1, 1, 1, window + 1, 2, T]:
            n = min(max(n, 1), T - at)
            if n <= 0:
                break
            pos, slot = _i32(list(range(at, at + n))), _i32([r] * n)
            if n > 1:
                ops.kv_write(qk[at:at + n], k_off, k_off, pool, table, pos, slot, 0, page, G, hd, 0)
            # a single row is a decode step: the kernel takes the row's own key from the row and writes the page itself
            got.append(ops.paged_attention_general(qk[at:at + n], H, hd, 0, pool, table, pos, slot, 0, page, G, 0.6,
                                                   window=window, slopes=slopes, q_temp=(0.8, 3), warps=1 + window % 4,
                                                   write_new=(k_off, k_off, None) if n == 1 else None))
            at += n
        got = torch.cat(got).double().cpu()
        tol = 1e-4 if dtype == torch.float32 else 2e-2
        assert got.shape == want.shape
        assert (got - want).abs().max() < tol * max(1.0, float(want.abs().max())), (r, float((got - want).abs().max()))


@pytest.mark.parametrize("hd,window,page,R", [(16, 21, 16, 3), (48, 7, 16, 1), (64, 100, 64, 4), (32, 64, 32, 2), (32, 1, 16, 2)])
def test_tensor_core_attention_of_portions_with_window_slopes_and_temperature(hd, window, page, R):
    """The tensor-core kernel for portions against the plain attention: three items of unequal length in one launch,
    each continuing a request at a position inside a window and inside a page; and the CUDA-core kernel on the
    same cache."""
    from fellm_b200 import ops
    G = 2
    H = G * R
    g = torch.Generator().manual_seed(hd + window)
    cfg = dict(heads=H, kv_heads=G, dim=hd, scale=0.4, mask=dict(size=window), q_temp=dict(coef=0.6, every=5))
    lens, done = [70, 1, 33], [window + 3, 2 * page - 1, 0]
    n_pages = [-(-(a + b) // page) for a, b in zip(lens, done)]
    pool = torch.zeros(sum(n_pages) + 1, 2, G * page * hd, dtype=torch.bfloat16, device=DEV)
    table = torch.full((3, max(n_pages)), -1, dtype=torch.int32, device=DEV)
    perm = torch.randperm(sum(n_pages), generator=g).to(torch.int32)
    at = 0
    for r in range(3):
        table[r, :n_pages[r]] = perm[at:at + n_pages[r]]
        at += n_pages[r]
    slopes = P.distance_slopes(H, torch.float64).float().to(DEV)
    rows, wants, pos, slot, starts, layer = [], [], [], [], [0], 1
    for r in range(3):
        T = lens[r] + done[r]
        qk = (torch.randn(T, (H + G) * hd + 8, generator=g) * 1.5).bfloat16()
        q, k = qk[:, :(H + G) * hd].float().split([H * hd, G * hd], 1)
        wants.append(_windowed_want(q, k, cfg)[done[r]:])
        dev = qk.to(DEV)
        if done[r]:
            ops.kv_write(dev[:done[r]], H * hd, H * hd, pool, table, _i32(list(range(done[r]))), _i32([r] * done[r]),
                         layer, page, G, hd, 0)
        rows.append(dev[done[r]:])
        pos += list(range(done[r], T))
        slot += [r] * lens[r]
        starts.append(starts[-1] + lens[r])
    qk_d = torch.cat(rows).contiguous()
    pos_d, slot_d = _i32(pos), _i32(slot)
    ops.kv_write(qk_d, H * hd, H * hd, pool, table, pos_d, slot_d, layer, page, G, hd, 0)
    got = ops.attention_prefill_general(qk_d, H, pool, table, pos_d, slot_d, _i32(starts), 3, max(lens), layer, 0.4,
                                        window=window, slopes=slopes, q_temp=(0.6, 5),
                                        values_are_keys=(G, page, hd)).double().cpu()
    want = torch.cat(wants)
    assert (got - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max())), float((got - want).abs().max())
    simt = ops.paged_attention_general(qk_d, H, hd, 0, pool, table, pos_d, slot_d, layer, page, G, 0.4, window=window,
                                       slopes=slopes, q_temp=(0.6, 5)).double().cpu()
    assert (simt - want).abs().max() < 2e-2 * max(1.0, float(want.abs().max()))


def _retention_want(q, k, v, decay, rot, base, dk):
    qr = P.rotate_half_partial(q.double(), rot, base) if rot else q.double()
    kr = (P.rotate_half_partial(k.double(), rot, base) if rot else k.double()) * dk ** -0.5
    return P.retention_scan(qr, kr, v.double(), torch.tensor(decay, dtype=torch.float64))


@pytest.mark.parametrize("H,dk,dv,rot", [(3, 20, 12, 8), (2, 32, 48, 32), (1, 64, 64, 16), (4, 8, 40, 0), (2, 128, 32, 64), (1, 200, 5, 6)])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_retention_scan(H, dk, dv, rot, dtype):
    """The scan in portions of 1, 2 and more tokens against the plain recurrence: key sizes on one lane, on several and
    no power of two, value sizes that do not fill a warp, rotation of all, part and none of the key; a portion
    starts at any position (the angles follow the positions, not the rows)."""
    from fellm_b200 import ops
    T = 45
    g = torch.Generator().manual_seed(H * 100 + dk)
    q, k, v = (torch.randn(T, H, d_, generator=g).to(dtype).float() for d_ in (dk, dk, dv))
    decay = [1.0 - 0.5 ** (1 + 2 * h) for h in range(H)]
    base = 50.0
    want = _retention_want(q, k, v, decay, rot, base, dk).reshape(T, H * dv)
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), torch.zeros(T, 4), v.reshape(T, -1)], 1).to(dtype).to(DEV)
    k_off, v_off = H * dk, 2 * H * dk + 4
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV) if rot else None
    state = torch.full((3, H, dk, dv), 9.0, device=DEV)
    state[1].zero_()
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    at = 0
    for n in [2, 1, 1, 17, 2, 22]:
        got = ops.retention_scan(qkv[at:at + n], k_off, v_off, _i32(list(range(at, at + n))), inv_freq, rot, dec, dk ** -0.5,
                                 state, _i32([0, n]), _i32([1]), 1, H, dk, dv)
        err = (got.double().cpu() - want[at:at + n]).abs().max()
        assert err < 3e-5 * max(1.0, float(want.abs().max())), (at, n, float(err))
        at += n
    assert float(state[0].min()) == 9.0 and float(state[2].max()) == 9.0       # the neighbours' slots are untouched


@pytest.mark.parametrize("H,dk,dv,rot", [(3, 20, 12, 8), (2, 32, 48, 32), (1, 64, 64, 16), (2, 128, 128, 64), (1, 200, 5, 6), (2, 8, 150, 0)])
def test_retention_in_blocks_of_tokens(H, dk, dv, rot):
    """The blocked form against the plain recurrence and against the scan: two requests in one launch with portions of
    unequal length (1, 2, 63, 64, 65 and 200 tokens among them: inside a block, on its edge, over several blocks), each
    going on from the state and the position its last portion left; the states end equal to the scan's."""
    from fellm_b200 import ops
    T = [330, 333]
    g = torch.Generator().manual_seed(H * 10 + dk)
    decay = [1.0 - 0.5 ** (2 + 3 * h) for h in range(H)]
    base = 300.0
    inv_freq = torch.tensor([base ** (-2.0 * i / rot) for i in range(rot // 2)], dtype=torch.float64).float().to(DEV) if rot else None
    dec = torch.tensor(decay, dtype=torch.float32, device=DEV)
    k_off, v_off = H * dk, 2 * H * dk + 4
    rows, wants = [], []
    for r in range(2):
        q, k, v = (torch.randn(T[r], H, d_, generator=g) for d_ in (dk, dk, dv))
        wants.append(_retention_want(q, k, v, decay, rot, base, dk).reshape(T[r], H * dv))
        rows.append(torch.cat([q.reshape(T[r], -1), k.reshape(T[r], -1), torch.zeros(T[r], 4), v.reshape(T[r], -1)], 1).to(DEV))
    state = torch.full((4, H, dk, dv), 7.0, device=DEV)
    state[1].zero_()
    state[3].zero_()
    scan_state = state.clone()
    cuts = [[64, 1, 200, 65], [2, 63, 130, 138]]
    at = [0, 0]
    for step in range(4):
        n = [cuts[0][step], cuts[1][step]]
        p = torch.cat([rows[r][at[r]:at[r] + n[r]] for r in range(2)]).contiguous()
        pos = _i32(list(range(at[0], at[0] + n[0])) + list(range(at[1], at[1] + n[1])))
        starts, slots = _i32([0, n[0], n[0] + n[1]]), _i32([3, 1])
        got = ops.retention_chunked(p, k_off, v_off, pos, inv_freq, rot, dec, dk ** -0.5, state, starts, slots, 2, max(n), H, dk, dv)
        ref = ops.retention_scan(p, k_off, v_off, pos, inv_freq, rot, dec, dk ** -0.5, scan_state, starts, slots, 2, H, dk, dv)
        want = torch.cat([wants[r][at[r]:at[r] + n[r]] for r in range(2)])
        scale = max(1.0, float(want.abs().max()))
        assert (got.double().cpu() - want).abs().max() < 5e-5 * scale, (step, float((got.double().cpu() - want).abs().max()))
        assert (got - ref).abs().max() < 5e-5 * scale
        at = [at[0] + n[0], at[1] + n[1]]
    assert (state - scan_state).abs().max() < 5e-5 * max(1.0, float(scan_state.abs().max()))
    assert float(state[0].min()) == 7.0 and float(state[2].max()) == 7.0       # the neighbours' slots are untouched


def test_retention_keeps_a_far_write_and_forgets_by_its_decay():
    """Head 0 does not decay: what token 0 wrote is read back unchanged 600 tokens later.  Head 1 halves its state
    every token: the same read gives 2^-600, nothing."""
    from fellm_b200 import ops
    T, dk, dv = 601, 32, 16
    q = torch.zeros(T, 2, dk)
    k = torch.zeros(T, 2, dk)
    for t in range(1, T):
        k[t, :, 1 + t % (dk - 1)] = 1.0                     # never channel 0 again
    k[0, :, 0] = 1.0
    q[:, :, 1] = 1.0
    q[T - 1] = 0
    q[T - 1, :, 0] = 1.0
    v = torch.randn(T, 2, dv, generator=torch.Generator().manual_seed(1))
    qkv = torch.cat([q.reshape(T, -1), k.reshape(T, -1), v.reshape(T, -1)], 1).to(DEV)
    state = torch.zeros(1, 2, dk, dv, device=DEV)
    got = ops.retention_scan(qkv, 2 * dk, 4 * dk, _i32(list(range(T))), None, 0, torch.tensor([1.0, 0.5], device=DEV), 1.0,
                             state, _i32([0, T]), _i32([0]), 1, 2, dk, dv).cpu().view(T, 2, dv)
    assert (got[T - 1, 0] - v[0, 0]).abs().max() < 1e-5
    assert got[T - 1, 1].abs().max() < 1e-30


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("T,d,ff,E,top", [(1, 64, 24, 4, 2), (3, 96, 40, 5, 1), (70, 72, 9, 7, 3), (700, 128, 56, 6, 6), (1300, 64, 32, 8, 2),
                                          (300, 64, 24, 1, 1), (400, 72, 16, 2, 2)])
def test_routed_experts_from_logits_to_the_weighted_sum(dtype, T, d, ff, E, top):
    """Routing, the device-side plan, both grouped products and the combine against the plain mixture.  Expert e's
    down projection is scaled by 3^e: a row sent to the wrong expert, or weighted by the wrong score, is far off.
    1,300 tokens x 2 choices are more pairs than one tile of the plan holds; one or two small experts are fewer weight rows
    than a tile of the tensor-core product has."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(T + E)
    W = {"router": (torch.randn(E, d, generator=g) * 0.5).bfloat16().double()}
    for e in range(E):
        W[f"e{e}.gate"] = (torch.randn(ff, d, generator=g) * 0.2).bfloat16().double()
        W[f"e{e}.up"] = (torch.randn(ff, d, generator=g) * 0.2).bfloat16().double()
        W[f"e{e}.down"] = (torch.randn(d, ff, generator=g) * 0.1 * 3.0 ** e).bfloat16().double()
    h = torch.randn(T, d, generator=g).to(dtype)
    want = P.routed_experts(h.double(), W, "", dict(experts=E, top=top))
    z = (h.double() @ W["router"].T).float().to(DEV)
    idx, score = ops.moe_route(z, E, top)
    s = torch.softmax(z.double().cpu(), -1)
    ts, ti = torch.topk(s, top, -1)
    assert torch.equal(idx.cpu().long(), ti) and (score.cpu().double() - ts).abs().max() < 1e-6
    # the router's product and the routing in one launch give the same choice
    idx2, score2 = ops.moe_router(h.to(DEV), W["router"].to(dtype).to(DEV), top)
    same = (idx2 == idx).all(1)                                                  # (a close call may go the other way)
    assert float(same.float().mean()) > 0.99 and (score2 - score)[same].abs().max() < 1e-5
    x = torch.randn(T, d, generator=g)
    gate_up = [(W[f"e{e}.gate"].to(dtype).to(DEV), W[f"e{e}.up"].to(dtype).to(DEV)) for e in range(E)]
    dn = torch.stack([W[f"e{e}.down"] for e in range(E)]).to(dtype).to(DEV)
    modes = [("fma", 64, False)]
    if dtype == torch.bfloat16:
        modes.append(("mma", 64, False))
        if ff % 8 == 0:
            modes += [("mma", 64, True), ("umma", 128, True)]
    for mode, row_tile, inter in modes:
        plan = ops.moe_plan(idx, E, row_tile)
        srt, place = plan.sorted.cpu().long(), plan.place_of.cpu().long()
        flat = idx.cpu().long().reshape(-1)
        assert torch.equal(torch.sort(srt).values, torch.arange(T * top)) and torch.equal(srt[place], torch.arange(T * top))
        assert bool((flat[srt][1:] >= flat[srt][:-1]).all())                    # sorted by expert
        n_tiles = int(plan.n_tiles.cpu())
        tab = plan.table.cpu()[:3 * n_tiles].view(n_tiles, 3)
        assert n_tiles <= plan.max_tiles and int(tab[:, 2].sum()) == T * top and int(tab[:, 2].max()) <= row_tile
        for e, r0, n in tab.tolist():
            assert bool((flat[srt][r0:r0 + n] == e).all())
        if inter:
            gu = torch.stack([ops.interleave_gate_up(a, b) for a, b in gate_up]).contiguous()
        else:
            gu = torch.stack([torch.cat([a, b]) for a, b in gate_up]).contiguous()
        ops.MOE_MMA = mode != "fma"
        try:
            a = ops.moe_gemm(h.to(DEV), gu, plan, gated=True, gather=True, interleaved=inter)
            y = ops.moe_gemm(a, dn, plan, gated=False, gather=False)
        finally:
            ops.MOE_MMA = True
        out = x.to(DEV).clone()
        ops.moe_combine(out, y, plan, score)
        ops.check_umma_status(DEV)
        tol = 1e-5 if dtype == torch.float32 else 2e-2
        err = (out.double().cpu() - x.double() - want).abs().max()
        assert err < tol * max(1.0, float(want.abs().max())), (mode, inter, float(err))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_a_token_of_the_mixture_does_not_depend_on_the_batch(dtype):
    """A token alone, among a few and among hundreds: bit for bit the same in float32 (one kernel, every sum in the
    order of K); in bfloat16 the step's size picks the kernel, and the results agree up to rounding."""
    from fellm_b200 import ops
    g = torch.Generator().manual_seed(9)
    d, ff, E, top = 64, 48, 5, 2
    gate = (torch.randn(E, ff, d, generator=g) * 0.2).to(dtype).to(DEV)
    up = (torch.randn(E, ff, d, generator=g) * 0.2).to(dtype).to(DEV)
    inter = dtype == torch.bfloat16
    gu = torch.stack([ops.interleave_gate_up(gate[e], up[e]) if inter else torch.cat([gate[e], up[e]]) for e in range(E)]).contiguous()
    dn = (torch.randn(E, d, ff, generator=g) * 0.2).to(dtype).to(DEV)
    h = torch.randn(300, d, generator=g).to(dtype).to(DEV)
    z = torch.randn(300, E, generator=g).to(DEV)

    def run(rows):
        idx, score = ops.moe_route(z[rows].contiguous(), E, top)
        plan = ops.moe_plan(idx, E, ops.moe_row_tile(idx.numel(), inter, True))
        y = ops.moe_gemm(ops.moe_gemm(h[rows].contiguous(), gu, plan, gated=True, gather=True, interleaved=inter), dn, plan,
                         gated=False, gather=False)
        out = torch.zeros(len(rows), d, device=DEV)
        return ops.moe_combine(out, y, plan, score)
    whole = run(list(range(300)))
    for rows in ([17], [5, 200, 17, 299], list(range(100, 171))):
        got = run(rows)
        if dtype == torch.float32:
            assert torch.equal(got, whole[rows])
        else:
            assert (got - whole[rows]).abs().max() < 2e-2 * float(whole.abs().max())


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


@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_whole_prompt(engines, name):
    T = 150
    got = U.run_cuts(engines(name), "a", U.tokens(name, T, 0), [T])
    d = U.distance(got, U.plain_logits(name, T, 0))
    assert d < U.LIMIT[engines.dtype], d


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_layers_one_by_one(engines, name):
    """The residual stream after every layer run against the plain implementation's."""
    from fellm_b200.models import model as M
    cfg, w = U.plain_model(name)
    toks = U.tokens(name, 40, 1)
    want = []
    P.forward(toks, w, cfg, want)
    want = torch.stack(want)
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


@pytest.mark.parametrize("name", ["A", "B", "D"])
def test_prompt_against_token_by_token(engines, name):
    T = 90
    eng = engines(name)
    toks = U.tokens(name, T, 2)
    whole = U.run_cuts(eng, "a", toks, [T])
    single = U.run_cuts(eng, "b", toks, [])
    if engines.dtype == "float32":
        # every sum's order is set by the model's sizes and the position, not by the cut
        assert torch.equal(single, whole)
    assert U.distance(single, whole) < U.LIMIT["bfloat16"]
    assert U.distance(single, U.plain_logits(name, T, 2)) < U.LIMIT[engines.dtype]


@pytest.mark.parametrize("name,cuts", [("A", [2, 2, 3, 17, 2, 21, 1, 1, 23, 2, 48]), ("B", [7, 2, 71, 2, 9, 64, 3]),
                                       ("C", [15, 2, 1, 16, 17, 2, 33]), ("D", [8, 2, 9, 1, 10, 65])])
def test_portions_of_many_sizes(engines, name, cuts):
    T = 170
    eng = engines(name)
    toks = U.tokens(name, T, 3)
    got = U.run_cuts(eng, "a", toks, cuts)
    assert U.distance(got, U.plain_logits(name, T, 3)) < U.LIMIT[engines.dtype]


@pytest.mark.parametrize("name", ["A", "B"])
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
    alone = engines(name)
    for i in plans:
        want = P.forward(plans[i][0], w, cfg)
        d = U.distance(torch.cat(got[i]), want)
        assert d < U.LIMIT[engines.dtype], (i, d)
        if engines.dtype == "float32" and i in (1, 3):
            assert torch.equal(torch.cat(got[i]), U.run_cuts(alone, f"alone{i}", plans[i][0], [len(plans[i][0])]))


def test_wide_model(engines):
    """Width 1,024, heads of 64 and 128, pages of 64 tokens: the sizes at which the products, the attention of portions
    and the experts' grouped products run on their tensor-core kernels; portions, then token by token, the window of
    100 passed in both."""
    name, T = "W", 150
    toks = U.tokens(name, T, 7)
    got = U.run_cuts(engines(name, page_tokens=64), "a", toks, [140, 2, 5])
    assert U.distance(got, U.plain_logits(name, T, 7)) < U.LIMIT[engines.dtype]


def test_long_decoding(engines):
    """420 tokens, most of them one by one: every window slides over decoded tokens, pages are given back on the way."""
    name, T = "A", 420
    toks = U.tokens(name, T, 5)
    got = U.run_cuts(engines(name, max_tokens=256), "a", toks, [20])
    assert U.distance(got, U.plain_logits(name, T, 5)) < U.LIMIT[engines.dtype]


def test_scaled_queries_and_keys_show_a_wrong_window(engines):
    """Attention weights scaled so that a softmax is nearly one-hot: a key let in from outside its window, the oldest
    key inside left out, a slope or a temperature step misplaced would change the logits far beyond rounding.  Also
    with the window at one position more and less than a page."""
    from fellm_b200.weights.safetensors_io import write_safetensors
    for n_case, window in enumerate([21, 15, 17] if engines.dtype == "float32" else [21]):
        cfg = copy.deepcopy(U.CFG_A)
        cfg["layers"][1]["mixer"]["mask"]["size"] = window
        cfg["layers"][1]["mixer"]["scale"] = 1.0
        cfg["layers"][2]["mixer"]["scale"] = 1.0
        _, w = U.plain_model("A")
        w = {n: t.clone() for n, t in w.items()}
        for n in ("l1.mix.q", "l1.mix.k", "l2.mix.q", "l2.mix.k"):
            w[n] = (w[n].float() * 20).bfloat16().double()
        folder = Path(U._tmp.name) / f"sharp_{engines.dtype}_{n_case}"
        folder.mkdir(exist_ok=True)
        (folder / "config.json").write_text(json.dumps(cfg))
        write_safetensors(folder / "model.safetensors", {n: t.bfloat16() for n, t in w.items()})
        eng = U.make_engine(str(folder), engines.dtype)
        toks = U.tokens("A", 80, 6)
        got = U.run_cuts(eng, "a", toks, [3, 2, 11, 1, 1, 30])
        want = P.forward(toks, w, cfg)
        # (scores this large carry more rounding into the softmax; a key wrongly seen or missed changes the logits by
        # parts in ten)
        assert U.distance(got, want) < 5 * U.LIMIT[engines.dtype], window


@pytest.mark.parametrize("seed", range(10))
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_configurations_drawn_at_random(seed, dtype):
    """Ten models of random shape, each under three regimes: the whole prompt, portions down to two tokens followed by
    single tokens, and two unequal requests sharing every step."""
    from fellm_b200.engine import StepItem
    from fellm_b200.weights import write_model_folder
    cfg = U.random_config(seed)
    folder = str(write_model_folder(Path(U._tmp.name) / f"random_{seed}", cfg, 500 + seed))
    _, w = U.load_folder(folder)
    eng = U.make_engine(folder, dtype, max_tokens=512)
    rng = np.random.default_rng(seed)
    T = 75
    toks = [int(t) for t in rng.integers(0, cfg["vocab"], T)]
    other = [int(t) for t in rng.integers(0, cfg["vocab"], 41)]
    want, want_other = P.forward(toks, w, cfg), P.forward(other, w, cfg)
    limit = U.LIMIT[dtype] * (3 if dtype == "bfloat16" else 1)      # (several passes of a loop add up their rounding)
    assert U.distance(U.run_cuts(eng, "whole", toks, [T]), want) < limit, cfg
    assert U.distance(U.run_cuts(eng, "cut", toks, [2, 17, 2, 3, 31]), want) < limit, cfg
    eng.add_request("a")
    eng.add_request("b")
    got_a, got_b, at_a, at_b = [], [], 0, 0
    sizes_a, sizes_b = [5, 1, 30, 2], [1, 1, 16, 7, 2]
    while at_a < T or at_b < len(other):
        items = []
        na = min(sizes_a.pop(0) if sizes_a else 1, T - at_a)
        nb = min(sizes_b.pop(0) if sizes_b else 1, len(other) - at_b)
        if na > 0:
            items.append(StepItem("a", toks[at_a:at_a + na], list(range(na))))
        if nb > 0:
            items.append(StepItem("b", other[at_b:at_b + nb], list(range(nb))))
        lg = eng.step(items)
        if na > 0:
            got_a.append(lg[:na].clone())
        if nb > 0:
            got_b.append(lg[max(na, 0):max(na, 0) + nb].clone())
        at_a, at_b = at_a + max(na, 0), at_b + max(nb, 0)
    eng.check_status()
    assert U.distance(torch.cat(got_a), want) < limit, cfg
    assert U.distance(torch.cat(got_b), want_other) < limit, cfg


@pytest.mark.parametrize("name", ["A", "B"])
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
            lg = P.forward(seq, w, cfg)[-1]
            top = torch.topk(lg, 2).values
            if int(lg.argmax()) != got[k]:
                assert float(top[0] - top[1]) < 1e-4 * float(lg.abs().max()), (k, got, int(lg.argmax()))
                break
            seq.append(got[k])
    assert all(s is not None for s in stats)


def test_command_line_runs_the_design(capsys):
    from fellm_b200 import cli
    folder = U.model_folder("A")
    assert cli.main(["inspect", "--model", folder]) == 0
    out = capsys.readouterr().out
    assert "architecture: Samusun" in out and "l0.mlp.e3.up" in out
    assert cli.main(["run", folder, "--prompt", "5 17 3 9 100", "--max-tokens", "6", "--temperature", "0", "--repetition-penalty", "1.0",
                     "--dtype", "float32", "--page-tokens", "16", "-c", "256", "--kv-device-budget", "4194304"]) == 0
    toks = [int(t) for t in capsys.readouterr().out.split()]
    cfg, w = U.plain_model("A")
    seq = [5, 17, 3, 9, 100]
    for t in toks:
        lg = P.forward(seq, w, cfg)[-1]
        top = torch.topk(lg, 2).values
        assert int(lg.argmax()) == t or float(top[0] - top[1]) < 1e-4 * float(lg.abs().max())
        seq.append(t)
    assert len(toks) == 6


def test_bfloat16_generation_runs_through_the_entry_point():
    from fellm_b200.engine import GenParams
    eng = U.make_engine("C", "bfloat16", cuda_graphs=True, n_ubatch=16, n_batch=64)
    out = list(eng.generate(U.tokens("C", 50, 30), GenParams.greedy(20)))
    assert len(out) == 20 and all(0 <= t < U.CFG_C["vocab"] for t in out)
