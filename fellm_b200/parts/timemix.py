"""Time mixing with a decaying matrix state and a bonus for the current token (the RWKV family's
recurrence).

    h' = the previous token's input (zeros before the first); each of r, k, v, g, w reads its own mix
    h + (h' - h) mu_s
    r, k, v = W_r, W_k, W_v of their mixes (H heads of dk); gate = SiLU(W_g mix_g)
    decay  w = exp(-exp(W_w2 tanh(W_w1 mix_w) + w0)), per head and key channel
    per head:  o_t = (S + diag(u) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T
    o per head over its root mean square, heads side by side, times a weight [H dk], times the gate; W_o.

Kept per request, float32: the previous token's input [d] and S [H, dk, dk].  The decay's rank is read
from the tensors' shapes."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError, WeightError
from .base import FixedState, Mixer, ParamDecl, register_part
from .gated_delta import _pad_rows
from .linear import linear, linear_modules

MIXES = ("r", "k", "v", "g", "w")


@register_part("mixer", "time_mix")
class TimeMix(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, key_dim: int, norm_eps: float, fallback_rank: int = 16):
        super().__init__()
        self.size, self.H, self.dk, self.eps = int(size), int(heads), int(key_dim), float(norm_eps)
        if self.dk > ops.MAX_SCAN_KEY_DIM:
            raise ConfigError(f"time_mix: key size {self.dk} is above {ops.MAX_SCAN_KEY_DIM}")
        d, n, R = self.size, self.H * self.dk, int(fallback_rank)
        self.decls = {f"mu.{s}": ParamDecl((d,), role="vector", init=("uniform", 0.0, 1.0)) for s in MIXES}
        self.decls.update({
            "r.weight": ParamDecl((n, d)), "k.weight": ParamDecl((n, d), init=("normal", 0.05)),
            "v.weight": ParamDecl((n, d), init=("normal", 0.05)), "g.weight": ParamDecl((n, d)),
            "w1.weight": ParamDecl((-1, d), init=("normal", 0.1), fallback=(R, d)),
            "w2.weight": ParamDecl((n, -1), init=("normal", 0.3), fallback=(n, R)),
            "w0": ParamDecl((n,), role="vector", init=("uniform", -3.0, 0.0)),
            "u": ParamDecl((self.H, self.dk), role="vector", init=("normal", 0.5)),
            "norm.weight": ParamDecl((n,), role="vector", init=("uniform", 0.5, 1.5)),
            "o.weight": ParamDecl((d, n)),
        })

    def prepare(self):
        w = self.w
        w["mu"] = torch.stack([w.pop(f"mu.{s}") for s in MIXES], 0).contiguous()
        self.rank = w["w1.weight"].shape[0]
        if w["w2.weight"].shape[1] != self.rank:
            raise WeightError(f"time_mix: the decay's factors have ranks {self.rank} and {w['w2.weight'].shape[1]}")
        for name in ("r.weight", "k.weight", "v.weight", "g.weight", "w1.weight"):
            w[name] = _pad_rows(w[name])        # whole groups of output columns for the products' vector stores

    def cache_need(self):
        return [FixedState((self.size,)), FixedState((self.H, self.dk, self.dk))]

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a time_mix layer cannot run on another layer's state")
        shift_state, mat_state = cache
        w = self.w
        mixes = ops.token_shift_mix(xn, w["mu"], shift_state.states, ctx.item_start, shift_state.item_slot,
                                    ctx.n_items, ctx.max_item_rows)
        n = self.H * self.dk
        r = linear(mixes[0], w["r.weight"])[:, :n]
        k = linear(mixes[1], w["k.weight"])[:, :n]
        v = linear(mixes[2], w["v.weight"])[:, :n]
        g = linear(mixes[3], w["g.weight"])[:, :n]
        z = linear(mixes[4], w["w1.weight"], out_dtype=torch.float32)
        decay = ops.lowrank_expand(z[:, :self.rank], w["w2.weight"], w["w0"], f_in="tanh", f_out="exp_neg_exp")
        o = ops.decay_bonus_scan(r, k, v, decay, w["u"], mat_state.states, ctx.item_start, mat_state.item_slot,
                                 ctx.n_items, self.H, self.dk, max_item_rows=ctx.max_item_rows)
        y = ops.head_norm_gate(o, w["norm.weight"], True, g, "silu", self.eps, self.H, self.dk, xn.dtype)
        linear(y, w["o.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        w = self.w
        return [w["r.weight"], w["k.weight"], w["v.weight"], w["g.weight"], w["w1.weight"], w["o.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("recurrent", None)]
