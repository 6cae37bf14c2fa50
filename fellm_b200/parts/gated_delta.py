"""Gated delta rule mixer (the recurrence of FeLLM's GatedDeltaNet layers,
crates/fellm-model/src/graph.rs:792-806, which keep a convolution history and a matrix per request).

    q, k = W_q h, W_k h (G heads of dk);  v = W_v h (H heads of dv);  head h reads q/k head h // (H / G)
    each of q, k, v: a short causal convolution per channel, then SiLU
    q, k: unit vectors per head (x / sqrt(sum x^2 + 1e-6)); q also times dk^(-1/2)
    beta = sigmoid(W_b h), one per head
    decay 'head':     g = exp(-exp(A_log) softplus(W_a h + dt_bias)), one per head
    decay 'channel':  g = exp(-exp(A_log) softplus(W_a2 (W_a1 h) + dt_bias)), one per head and key channel
    per head:  S <- g S;  u = beta (v - S^T k);  S <- S + k u^T;  o = S^T q
    o per head over its root mean square, times a weight [dv] shared by the heads, times the output gate:
        gate 'silu': SiLU(W_g h);  gate 'sigmoid_lowrank': sigmoid(W_g2 (W_g1 h))
    then W_o.

What is kept per request: the last taps-1 inputs of the convolutions, and S [H, dk, dv], both float32.
The ranks of the low-rank projections are read from the tensors' shapes.
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError, WeightError
from .base import FixedState, Mixer, ParamDecl, register_part
from .linear import linear, linear_modules


def _pad_rows(w: torch.Tensor, multiple: int = 16) -> torch.Tensor:
    """Rows of zeros up to a multiple: the products' vector stores want whole groups of columns."""
    n = w.shape[0]
    extra = -n % multiple
    if not extra:
        return w.contiguous()
    return torch.cat([w, torch.zeros((extra, w.shape[1]), dtype=w.dtype, device=w.device)], 0).contiguous()


def stack_rows(mats):
    """One matrix of several projections that read the same input (float32 if their dtypes differ), padded to a
    multiple of 16 rows; returns it and each projection's first row."""
    dt = mats[0].dtype if all(m.dtype == mats[0].dtype for m in mats) else torch.float32
    offs, at = [], 0
    for m in mats:
        offs.append(at)
        at += m.shape[0]
    return _pad_rows(torch.cat([m.to(dt) for m in mats], 0)), offs


@register_part("mixer", "gated_delta")
class GatedDelta(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, kv_heads: int, key_dim: int, value_dim: int, taps: int,
                 norm_eps: float, decay: str = "head", gate: str = "silu", fallback_rank: int = 16):
        super().__init__()
        self.size, self.H, self.G = int(size), int(heads), int(kv_heads)
        self.dk, self.dv, self.taps, self.eps = int(key_dim), int(value_dim), int(taps), float(norm_eps)
        if self.H % self.G:
            raise ConfigError(f"gated_delta: {self.H} heads are not a multiple of {self.G} key heads")
        if decay not in ("head", "channel") or gate not in ("silu", "sigmoid_lowrank"):
            raise ConfigError(f"gated_delta: unknown decay {decay!r} or gate {gate!r}")
        if not 1 <= self.taps <= ops.MAX_CONV_TAPS:
            raise ConfigError(f"gated_delta: {self.taps} convolution taps are outside 1..{ops.MAX_CONV_TAPS}")
        if self.dk > ops.MAX_SCAN_KEY_DIM:
            raise ConfigError(f"gated_delta: key size {self.dk} is above {ops.MAX_SCAN_KEY_DIM}")
        self.decay, self.gate = decay, gate
        d, H, G, dk, dv, L, R = self.size, self.H, self.G, self.dk, self.dv, self.taps, int(fallback_rank)
        taps_init = ("normal", 0.5)
        self.decls = {
            "q.weight": ParamDecl((G * dk, d)), "k.weight": ParamDecl((G * dk, d)), "v.weight": ParamDecl((H * dv, d)),
            "q.conv": ParamDecl((G * dk, L), role="vector", init=taps_init),
            "k.conv": ParamDecl((G * dk, L), role="vector", init=taps_init),
            "v.conv": ParamDecl((H * dv, L), role="vector", init=taps_init),
            "b.weight": ParamDecl((H, d), init=("normal", 0.1)),
            "A_log": ParamDecl((H,), role="vector", init=("uniform", -2.0, 0.5)),
            "norm.weight": ParamDecl((dv,), role="vector", init=("uniform", 0.5, 1.5)),
            "o.weight": ParamDecl((d, H * dv)),
        }
        if decay == "head":
            self.decls["a.weight"] = ParamDecl((H, d), init=("normal", 0.1))
            self.decls["dt_bias"] = ParamDecl((H,), role="vector", init=("uniform", -1.0, 1.0))
        else:
            self.decls["a1.weight"] = ParamDecl((-1, d), init=("normal", 0.1), fallback=(R, d))
            self.decls["a2.weight"] = ParamDecl((H * dk, -1), init=("normal", 0.2), fallback=(H * dk, R))
            self.decls["dt_bias"] = ParamDecl((H * dk,), role="vector", init=("uniform", -1.0, 1.0))
        if gate == "silu":
            self.decls["g.weight"] = ParamDecl((H * dv, d))
        else:
            self.decls["g1.weight"] = ParamDecl((-1, d), init=("normal", 0.1), fallback=(R, d))
            self.decls["g2.weight"] = ParamDecl((H * dv, -1), init=("normal", 0.2), fallback=(H * dv, R))

    def prepare(self):
        """Every projection that reads the mixer's input is one product: [q; k; v; (g); b; a or a1; (g1)], stored in
        float32 (the logits of beta and of the decay must not be rounded, and one launch is cheaper than two)."""
        w = self.w
        G, H, dk, dv = self.G, self.H, self.dk, self.dv
        self.n_conv = 2 * G * dk + H * dv
        mats = [w.pop("q.weight"), w.pop("k.weight"), w.pop("v.weight")]
        names = ["q", "k", "v"]
        if self.gate == "silu":
            mats.append(w.pop("g.weight"))
            names.append("g")
        mats.append(w.pop("b.weight"))
        names.append("b")
        if self.decay == "head":
            mats.append(w.pop("a.weight"))
            names.append("a")
        else:
            a1, a2 = w.pop("a1.weight"), w["a2.weight"]
            if a1.shape[0] != a2.shape[1]:
                raise WeightError(f"gated_delta: the decay's factors have ranks {a1.shape[0]} and {a2.shape[1]}")
            mats.append(a1)
            names.append("a")
        if self.gate == "sigmoid_lowrank":
            g1, g2 = w.pop("g1.weight"), w["g2.weight"]
            if g1.shape[0] != g2.shape[1]:
                raise WeightError(f"gated_delta: the gate's factors have ranks {g1.shape[0]} and {g2.shape[1]}")
            mats.append(g1)
            names.append("g")
        w["in.weight"], offs = stack_rows(mats)
        self.off = dict(zip(names, offs))
        self.rows = {n: m.shape[0] for n, m in zip(names, mats)}
        w["taps"] = torch.cat([w.pop("q.conv"), w.pop("k.conv"), w.pop("v.conv")], 0).contiguous()

    def cache_need(self):
        return [FixedState((self.taps - 1, 2 * self.G * self.dk + self.H * self.dv)),
                FixedState((self.H, self.dk, self.dv))]

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a gated_delta layer cannot run on another layer's state")
        conv_state, mat_state = cache
        w, off = self.w, self.off
        H, G, dk, dv = self.H, self.G, self.dk, self.dv
        p = linear(xn, w["in.weight"], out_dtype=torch.float32)            # [T, q | k | v | (g) | b | a or a1 | (g1)] float32
        qkv = ops.causal_conv_act(p[:, :self.n_conv], w["taps"], conv_state.states, ctx.item_start,
                                  conv_state.item_slot, ctx.n_items, ctx.max_item_rows, act="silu")
        gch = None
        if self.decay == "channel":
            gch = ops.lowrank_expand(p[:, off["a"]:off["a"] + self.rows["a"]], w["a2.weight"], w["dt_bias"],
                                     f_out="decay_softplus", rate=w["A_log"], per=dk)
        o = ops.delta_scan(qkv, off["k"], off["v"], p, off["b"], off["a"], w["A_log"],
                           None if gch is not None else w["dt_bias"], gch, mat_state.states, ctx.item_start,
                           mat_state.item_slot, ctx.n_items, H, G, dk, dv, max_item_rows=ctx.max_item_rows)
        if self.gate == "silu":
            gate, act = p[:, off["g"]:off["g"] + H * dv], "silu"
        else:
            gate, act = ops.lowrank_expand(p[:, off["g"]:off["g"] + self.rows["g"]], w["g2.weight"]), "sigmoid"
        y = ops.head_norm_gate(o, w["norm.weight"], False, gate, act, self.eps, H, dv, xn.dtype)
        linear(y, w["o.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["in.weight"], self.w["o.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("recurrent", None)]
