"""A plain, slow implementation of the Samusun design in PyTorch on the CPU: one function per
mechanism, token by token where a mechanism is recurrent, no cache, no batching, no kernels.
It shares no code with fellm_b200: the tests compare the engine with it.

Notation: d model width, H heads, G key/value heads, dk key size, dv value size, T tokens, E experts.
Weights are a dict {tensor name: tensor}; everything is computed in the dtype of the weights handed
in (float64 for the oracle).  `cfg` is the parsed config.json of the model.
"""
from __future__ import annotations

import math

import torch
import torch.nn.functional as F


def rms_unit(x, eps):
    """x over its root mean square along the last axis, eps under the root."""
    return x / torch.sqrt((x * x).mean(-1, keepdim=True) + eps)


def rms_norm(x, w, eps):
    return rms_unit(x, eps) * w


def query_temperature(T, coef, every, dtype):
    """Factor of the query at positions 0..T-1: 1 + coef ln(floor((p + 1) / every) + 1)."""
    p = torch.arange(T)
    return (1.0 + coef * torch.log(((p + 1) // every + 1).to(dtype))).to(dtype)


def distance_slopes(H, dtype):
    """slope of head h = 2^(-8 (h + 1) / H)."""
    return torch.tensor([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=dtype)


def windowed_attention(q, k, v, scale, window, slopes):
    """q [T, H, dk]; k [T, G, dk]; v [T, G, dv]; query head h reads key/value head h // (H / G).
    score(i, j) = q_i . k_j scale - slope_h (i - j) for 0 <= i - j < window, softmax over those."""
    T, H, _ = q.shape
    G = k.shape[1]
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for h in range(H):
        g = h // (H // G)
        for i in range(T):
            lo = max(0, i - window + 1)
            s = (k[lo:i + 1, g] @ q[i, h]) * scale
            s = s - slopes[h] * (i - torch.arange(lo, i + 1)).to(q.dtype)
            p = torch.softmax(s, 0)
            out[i, h] = p @ v[lo:i + 1, g]
    return out


def attention_mixer(h, W, p, m):
    """The 'attention' mixer: biased q, k and output projections, the keys are also the values, no rotation,
    a query temperature by position, a bias by distance, a sliding window."""
    H, G, dk = m["heads"], m["kv_heads"], m["dim"]
    T = h.shape[0]
    q = (h @ W[p + "q"].T + W[p + "q.b"]).view(T, H, dk)
    k = (h @ W[p + "k"].T + W[p + "k.b"]).view(T, G, dk)
    q = q * query_temperature(T, m["q_temp"]["coef"], m["q_temp"]["every"], h.dtype)[:, None, None]
    o = windowed_attention(q, k, k, m["scale"], m["mask"]["size"], distance_slopes(H, h.dtype))
    return o.reshape(T, -1) @ W[p + "o"].T + W[p + "o.b"]


def rotate_half_partial(x, dims, base):
    """x [T, H, dk]: the first `dims` elements of every head are rotated, element i paired with i + dims/2,
    angle = position * base^(-2i/dims); the other elements pass."""
    T = x.shape[0]
    half = dims // 2
    f = torch.tensor([base ** (-2.0 * i / dims) for i in range(half)], dtype=x.dtype)
    a = torch.arange(T, dtype=x.dtype)[:, None] * f[None, :]
    c, s = torch.cos(a)[:, None, :], torch.sin(a)[:, None, :]
    u, v = x[..., :half], x[..., half:dims]
    return torch.cat([u * c - v * s, v * c + u * s, x[..., dims:]], -1)


def retention_scan(q, k, v, decay):
    """Per head: S_t = decay_h S_(t-1) + k_t v_t^T; o_t = S_t^T q_t.  q, k [T, H, dk]; v [T, H, dv]."""
    T, H, dk = q.shape
    S = torch.zeros(H, dk, v.shape[-1], dtype=q.dtype)
    out = torch.zeros(T, H, v.shape[-1], dtype=q.dtype)
    for t in range(T):
        S = S * decay[:, None, None] + torch.einsum("hk,hv->hkv", k[t], v[t])
        out[t] = torch.einsum("hkv,hk->hv", S, q[t])
    return out


def retention_mixer(h, W, p, m, eps):
    """The 'retention' mixer: rotary q and k, k over sqrt(dk), the decaying sum, every head's read-out over its
    root mean square, a SiLU gate, the output projection."""
    H, dk, dv = m["heads"], m["dim"], m["vdim"]
    T = h.shape[0]
    q = rotate_half_partial((h @ W[p + "q"].T).view(T, H, dk), m["rot"]["dims"], m["rot"]["base"])
    k = rotate_half_partial((h @ W[p + "k"].T).view(T, H, dk), m["rot"]["dims"], m["rot"]["base"]) * dk ** -0.5
    v = (h @ W[p + "v"].T).view(T, H, dv)
    o = retention_scan(q, k, v, torch.tensor(m["decay"], dtype=h.dtype))
    o = rms_unit(o, eps).reshape(T, H * dv) * F.silu(h @ W[p + "g"].T)
    return o @ W[p + "o"].T


def gated_ff(h, w_gate, w_up, w_down):
    return (F.silu(h @ w_gate.T) * (h @ w_up.T)) @ w_down.T


def routed_experts(h, W, p, router):
    """Scores = softmax of the router's logits over all experts; each token takes its `top` best experts, weighted
    by their scores as they are."""
    s = torch.softmax(h @ W[p + "router"].T, -1)
    top_s, top_e = torch.topk(s, router["top"], dim=-1)
    out = torch.zeros_like(h)
    for t in range(h.shape[0]):
        for sc, e in zip(top_s[t], top_e[t]):
            q = f"{p}e{int(e)}."
            out[t] = out[t] + sc * gated_ff(h[t:t + 1], W[q + "gate"], W[q + "up"], W[q + "down"])[0]
    return out


def feed_forward(h, W, p, mlp):
    if mlp["kind"] == "dense":
        return gated_ff(h, W[p + "gate"], W[p + "up"], W[p + "down"])
    return routed_experts(h, W, p, mlp["router"])


def layer_order(cfg):
    """[(layer, pass number when the entry opens a pass of the loop, else None)]."""
    n = len(cfg["layers"])
    loop = cfg.get("loop")
    if not loop:
        return [(i, None) for i in range(n)]
    a, b, times = loop["start"], loop["stop"], loop["times"]
    order = [(i, None) for i in range(a)]
    for t in range(times):
        order += [(i, t if i == a else None) for i in range(a, b)]
    return order + [(i, None) for i in range(b, n)]


def forward(tokens, W, cfg, layers_out=None):
    """tokens: list of ids of one sequence -> logits [T, vocab].  layers_out: a list that receives the residual
    stream after every layer run."""
    eps = cfg["norm"]["eps"]
    x = W["embed"][torch.tensor(tokens)] * cfg["embedding"]["scale"]
    for i, opens in layer_order(cfg):
        L = cfg["layers"][i]
        p = f"l{i}."
        if opens is not None:
            x = x + W["loop.step"][opens]
        h = rms_norm(x, W[p + "norm1"], eps)
        if L["type"] == "attention":
            y = attention_mixer(h, W, p + "mix.", L["mixer"])
        else:
            y = retention_mixer(h, W, p + "mix.", L["mixer"], eps)
        if L.get("mlp") is not None:
            y = y + feed_forward(h, W, p + "mlp.", L["mlp"])
        x = x + y
        if layers_out is not None:
            layers_out.append(x.clone())
    z = rms_norm(x, W["final.norm"], eps) @ W["head"].T * cfg["logit_scale"]
    cap = cfg["logit_softcap"]
    return cap * torch.tanh(z / cap)
