"""Retention mixer: linear attention with a fixed decay per head, no softmax and no denominator.

    q, k = W_q h, W_k h (H heads of dk);  v = W_v h (H heads of dv);  no biases
    q and k are rotated by position (the position part: the first rot_dim elements of a head, pairs (i, i + rot_dim/2)
    or (2i, 2i+1) as the part says; the other elements pass); k then times dk^(-1/2)
    per head:  S_t = decay_h S_(t-1) + k_t v_t^T;  o_t = S_t^T q_t
    o per head over its root mean square (no weight), heads side by side, times SiLU(W_g h); then W_o.

Kept per request, float32: S [H, dk, dv], zero when the request starts.  Float32 in both engines: the angles and the
rotation, the scaling of k, the decay, the state and its read-out, the unit norm.  The four projections are one
product whose result is stored in float32, so that nothing that enters the recurrence is rounded to bfloat16 again.
Token by token the recurrence is the engine's scan (csrc/recurrent.cu); prompt portions of the bfloat16 engine run in
blocks of 64 tokens side by side (csrc/retention_chunk.cu).
"""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import FixedState, Mixer, ParamDecl, build_part, register_part
from .gated_delta import stack_rows
from .linear import linear, linear_modules


@register_part("mixer", "retention")
class Retention(Mixer):
    def __init__(self, *, dtype: str, size: int, heads: int, key_dim: int, value_dim: int, decay, norm_eps: float,
                 position, key_scale=None):
        """`decay`: one factor per head.  `position`: a PartSpec of the 'position' category (rotary with the
        'split_half' pairing, or none).  `key_scale`: what the rotated keys are multiplied by (None: dk^-1/2)."""
        super().__init__()
        self.size, self.H, self.dk, self.dv = int(size), int(heads), int(key_dim), int(value_dim)
        self.eps = float(norm_eps)
        self.decay = [float(g) for g in decay]
        if len(self.decay) != self.H:
            raise ConfigError(f"retention: {len(self.decay)} decays for {self.H} heads")
        if self.dk > ops.MAX_SCAN_KEY_DIM:
            raise ConfigError(f"retention: key size {self.dk} is above {ops.MAX_SCAN_KEY_DIM}")
        self.position = build_part("position", position, dtype)
        self.rot_dim = 0
        if self.position.inv_freq is not None:
            self.rot_dim = int(getattr(self.position, "rot_dim", self.dk))
            if self.position.pairing != "split_half":
                raise ConfigError("retention: the rotation pairs element i with i + rot_dim/2 ('split_half')")
            if self.rot_dim % 2 or not 2 <= self.rot_dim <= self.dk:
                raise ConfigError(f"retention: rotary dimension {self.rot_dim} must be even and within the key size {self.dk}")
        self.key_scale = self.dk ** -0.5 if key_scale is None else float(key_scale)
        d, H, dk, dv = self.size, self.H, self.dk, self.dv
        self.decls = {"q.weight": ParamDecl((H * dk, d)), "k.weight": ParamDecl((H * dk, d)),
                      "v.weight": ParamDecl((H * dv, d)), "g.weight": ParamDecl((H * dv, d)),
                      "o.weight": ParamDecl((d, H * dv))}

    def prepare(self):
        w = self.w
        w["in.weight"], offs = stack_rows([w.pop("q.weight"), w.pop("k.weight"), w.pop("v.weight"), w.pop("g.weight")])
        self.off = dict(zip("qkvg", offs))
        dev = w["in.weight"].device
        w["decay"] = torch.tensor(self.decay, dtype=torch.float64).to(torch.float32).to(dev)
        self.position.to(dev)

    def cache_need(self):
        return FixedState((self.H, self.dk, self.dv))

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a retention layer cannot run on another layer's state")
        w, off, H, dk, dv = self.w, self.off, self.H, self.dk, self.dv
        p = linear(xn, w["in.weight"], out_dtype=torch.float32)             # [T, q | k | v | g] float32
        if xn.dtype == torch.bfloat16 and ops.RETENTION_CHUNKED and ctx.max_item_rows >= ops.RETENTION_CHUNK_MIN_ROWS:
            # portions of prompts in the bfloat16 engine: blocks of 64 tokens side by side (float32 arithmetic, another
            # order of the sums than the scan's; the 32-bit engine keeps the scan and the same bits under every cut)
            o = ops.retention_chunked(p, off["k"], off["v"], ctx.positions, self.position.inv_freq, self.rot_dim, w["decay"],
                                      self.key_scale, cache.states, ctx.item_start, cache.item_slot, ctx.n_items,
                                      ctx.max_item_rows, H, dk, dv)
        else:
            o = ops.retention_scan(p, off["k"], off["v"], ctx.positions, self.position.inv_freq, self.rot_dim, w["decay"],
                                   self.key_scale, cache.states, ctx.item_start, cache.item_slot, ctx.n_items, H, dk, dv,
                                   max_item_rows=ctx.max_item_rows)
        y = ops.head_norm_gate(o, None, False, p[:, off["g"]:off["g"] + H * dv], "silu", self.eps, H, dv, xn.dtype)
        linear(y, w["o.weight"], out=out, accumulate=True)
        return out

    def weight_order(self):
        return [self.w["in.weight"], self.w["o.weight"]]

    def kernel_modules(self, dtype):
        return linear_modules(dtype) + [("recurrent", None)] + ([("retention_chunk", None)] if dtype == "bfloat16" else [])
