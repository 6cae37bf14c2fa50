"""A plain, slow implementation of the Robazen design in PyTorch on the CPU: one function per
mechanism, token by token where a mechanism is recurrent, no cache, no batching, no kernels.
It shares no code with fellm_b200: the tests compare the engine with it.

Notation: d model width, H heads, G key/value heads, dk key size, dv value size, T tokens.
Weights are a dict {tensor name: tensor}; `dt` is the dtype everything is computed in
(float64 for the oracle; float32 to imitate the engine's 32-bit path).
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def dyt_norm(x, w, b, alpha):
    """Dynamic Tanh: no statistics, y = tanh(alpha x) w + b."""
    return torch.tanh(alpha * x) * w + b


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def causal_short_conv(x, taps):
    """x [T, C], taps [C, L]; out[t, c] = sum_j taps[c, j] x[t - (L-1) + j, c], zeros before t = 0."""
    T, C = x.shape
    L = taps.shape[1]
    xp = torch.cat([torch.zeros(L - 1, C, dtype=x.dtype), x], 0)
    out = torch.zeros_like(x)
    for j in range(L):
        out = out + xp[j:j + T] * taps[:, j]
    return out


def delta_rule_scan(q, k, v, beta, g):
    """Gated delta rule per head.  q, k [T, H, dk]; v [T, H, dv]; beta [T, H]; g [T, H] or [T, H, dk]
    (decay per head, or per head and key channel).  S [dk, dv] starts at zero; per token:
    S = g S; u = beta (v - S^T k); S = S + k u^T; o = S^T q."""
    T, H, dk = q.shape
    dv = v.shape[-1]
    S = torch.zeros(H, dk, dv, dtype=q.dtype)
    out = torch.zeros(T, H, dv, dtype=q.dtype)
    for t in range(T):
        gt = g[t]
        S = S * (gt[:, None, None] if gt.dim() == 1 else gt[:, :, None])
        u = beta[t][:, None] * (v[t] - torch.einsum("hkv,hk->hv", S, k[t]))
        S = S + torch.einsum("hk,hv->hkv", k[t], u)
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def gated_delta_mixer(h, W, p, cfg, eps, channelwise):
    """The 'delta' (channelwise=False) and 'channel_delta' (True) mixers.  h [T, d]."""
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = F.silu(causal_short_conv(h @ W[p + "q"].T, W[p + "q.conv"])).view(T, G, dk)
    k = F.silu(causal_short_conv(h @ W[p + "k"].T, W[p + "k.conv"])).view(T, G, dk)
    v = F.silu(causal_short_conv(h @ W[p + "v"].T, W[p + "v.conv"])).view(T, H, dv)
    q = q / torch.sqrt((q * q).sum(-1, keepdim=True) + 1e-6) * dk ** -0.5
    k = k / torch.sqrt((k * k).sum(-1, keepdim=True) + 1e-6)
    rep = H // G
    q = q.repeat_interleave(rep, dim=1)
    k = k.repeat_interleave(rep, dim=1)
    beta = torch.sigmoid(h @ W[p + "b"].T)
    rate = torch.exp(W[p + "A_log"])                                   # [H]
    if channelwise:
        a = ((h @ W[p + "a1"].T) @ W[p + "a2"].T + W[p + "dt_bias"]).view(T, H, dk)
        g = torch.exp(-rate[None, :, None] * F.softplus(a))
        gate = torch.sigmoid((h @ W[p + "g1"].T) @ W[p + "g2"].T)
    else:
        a = h @ W[p + "a"].T + W[p + "dt_bias"]
        g = torch.exp(-rate[None, :] * F.softplus(a))
        gate = F.silu(h @ W[p + "g"].T)
    o = delta_rule_scan(q, k, v, beta, g)                              # [T, H, dv]
    o = rms_unit(o, eps) * W[p + "norm"]
    o = o.reshape(T, H * dv) * gate
    return o @ W[p + "o"].T


def chunked_attention(h, W, p, cfg):
    """The left half of the 'parallel' mixer: grouped-query attention without positions, scores
    scaled, soft-capped, and masked to the query's own chunk of `mask.size` positions."""
    H, G, dk, dv = cfg["heads"], cfg["kv_heads"], cfg["dim"], cfg["vdim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T).view(T, H, dk)
    k = (h @ W[p + "k"].T).view(T, G, dk).repeat_interleave(H // G, dim=1)
    v = (h @ W[p + "v"].T).view(T, G, dv).repeat_interleave(H // G, dim=1)
    s = torch.einsum("ihk,jhk->hij", q, k) * cfg["scale"]
    cap = cfg.get("softcap")
    if cap:
        s = cap * torch.tanh(s / cap)
    i = torch.arange(T)[:, None]
    j = torch.arange(T)[None, :]
    size = cfg["mask"]["size"]
    visible = (j <= i) & (i // size == j // size)
    s = s.masked_fill(~visible, float("-inf"))
    a = torch.softmax(s, dim=-1)
    o = torch.einsum("hij,jhv->ihv", a, v)
    o = o * torch.sigmoid(h @ W[p + "g"].T)[:, :, None]
    return o.reshape(T, H * dv) @ W[p + "o"].T


def time_mix(h, W, p, cfg, eps):
    """The right half of the 'parallel' mixer: token shift with fixed mixes, a low-rank decay per
    key channel, the matrix state read BEFORE the decay with a bonus for the current token."""
    H, dk = cfg["heads"], cfg["dim"]
    T, d = h.shape
    prev = torch.cat([torch.zeros(1, d, dtype=h.dtype), h[:-1]], 0)

    def mix(s):
        return h + (prev - h) * W[p + "mu." + s]
    r = (mix("r") @ W[p + "r"].T).view(T, H, dk)
    k = (mix("k") @ W[p + "k"].T).view(T, H, dk)
    v = (mix("v") @ W[p + "v"].T).view(T, H, dk)
    gate = F.silu(mix("g") @ W[p + "g"].T)
    w = torch.exp(-torch.exp(torch.tanh(mix("w") @ W[p + "w1"].T) @ W[p + "w2"].T + W[p + "w0"])).view(T, H, dk)
    u = W[p + "u"]                                                      # [H, dk]
    S = torch.zeros(H, dk, dk, dtype=h.dtype)
    out = torch.zeros(T, H, dk, dtype=h.dtype)
    for t in range(T):
        kv = torch.einsum("hk,hv->hkv", k[t], v[t])
        out[t] = torch.einsum("hkv,hk->hv", S + u[:, :, None] * kv, r[t])
        S = w[t][:, :, None] * S + kv
    o = rms_unit(out, eps).reshape(T, H * dk) * W[p + "norm"] * gate
    return o @ W[p + "o"].T


def parallel_mixer(h, W, p, cfg, eps):
    left = chunked_attention(h, W, p + "left.", cfg["left"])
    right = time_mix(h, W, p + "right.", cfg["right"], eps)
    return 0.5 * (rms_unit(left, eps) * W[p + "left.out"] + rms_unit(right, eps) * W[p + "right.out"])


def dense_ff(h, W, p):
    return (F.silu(h @ W[p + "gate"].T) * (h @ W[p + "up"].T)) @ W[p + "down"].T


def layer_order(cfg):
    """[(layer index, pass number or None, first of its pass)] in running order."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None, False) for i in range(n)]
    order = [(i, None, False) for i in range(loop["start"])]
    for t in range(loop["times"]):
        for i in range(loop["start"], loop["stop"]):
            order.append((i, t, i == loop["start"]))
    return order + [(i, None, False) for i in range(loop["stop"], n)]


def forward(cfg, W, tokens, dt=torch.float64, keep_layers=False):
    """tokens: a list of ids of ONE sequence from its start.  Returns logits [T, vocab] (and the
    residual stream after every layer run)."""
    W = {n: (t.to(dt) if t.is_floating_point() else t) for n, t in W.items()}
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.as_tensor(tokens, dtype=torch.long)]
    x0 = x.clone()
    kept = []

    def norm(name, z):
        return dyt_norm(z, W[name], W[name + ".b"], W[name + ".alpha"])
    for i, t, first in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if first:
            x = torch.cat([x, x0], -1) @ W["loop.in"].T + W["loop.step"][t]
        hn = norm(p + "norm1", x)
        if L["type"] == "delta":
            m = gated_delta_mixer(hn, W, p + "mix.", L["mixer"], eps, False)
        elif L["type"] == "channel_delta":
            m = gated_delta_mixer(hn, W, p + "mix.", L["mixer"], eps, True)
        elif L["type"] == "parallel":
            m = parallel_mixer(hn, W, p + "mix.", L["mixer"], eps)
        else:
            raise ValueError(L["type"])
        x = x + m
        if L.get("mlp"):
            x = x + dense_ff(norm(p + "norm2", x), W, p + "mlp.")
        kept.append(x)
    logits = norm("final.norm", x) @ W["head"].T
    return (logits, torch.stack(kept)) if keep_layers else logits
