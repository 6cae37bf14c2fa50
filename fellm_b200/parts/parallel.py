"""Several mixers side by side on the same input: each branch's output is RMS-normed over the model
width with a plain weight of its own, and the mixer's result is the mean of the normed branches.
A branch is any registered mixer; what the branches keep between steps is kept side by side."""
from __future__ import annotations

import torch

from .. import ops
from ..config.errors import ConfigError
from .base import Mixer, ParamDecl, build_part, register_part


@register_part("mixer", "parallel")
class ParallelBranches(Mixer):
    def __init__(self, *, dtype: str, size: int, branches, norm_eps: float):
        """`branches`: a tuple of PartSpecs of the 'mixer' category.  Own tensors: out.<i>.weight [size]."""
        super().__init__()
        self.size, self.eps = int(size), float(norm_eps)
        if not 1 <= len(branches) <= 4:
            raise ConfigError(f"parallel mixer: {len(branches)} branches (1..4 are taken)")
        self.parts = [build_part("mixer", b, dtype) for b in branches]
        self.decls = {f"out.{i}.weight": ParamDecl((self.size,), role="vector", init=("uniform", 0.5, 1.5))
                      for i in range(len(self.parts))}
        self._spans = []
        at = 0
        for p in self.parts:
            need = p.cache_need()
            n = len(need) if isinstance(need, (list, tuple)) else (0 if need is None else 1)
            self._spans.append((at, n, isinstance(need, (list, tuple))))
            at += n

    def children(self):
        return list(self.parts)

    def cache_need(self):
        needs = []
        for p in self.parts:
            need = p.cache_need()
            needs += list(need) if isinstance(need, (list, tuple)) else ([] if need is None else [need])
        return needs

    def forward(self, xn, ctx, cache, out, reads_only=False):
        if reads_only:
            raise ConfigError("a parallel mixer cannot run on another layer's cache")
        outs = []
        bufs = torch.zeros((len(self.parts), xn.shape[0], self.size), dtype=torch.float32, device=out.device)   # one memset
        for p, (at, n, is_list), buf in zip(self.parts, self._spans, bufs):
            view = cache[at:at + n] if is_list else (cache[at] if n else None)
            p.forward(xn, ctx, view, buf)
            outs.append(buf)
        ops.branch_combine(out, outs, [self.w[f"out.{i}.weight"] for i in range(len(outs))], self.eps)
        return out

    def weight_order(self):
        return [w for p in self.parts for w in p.weight_order()]

    def kernel_modules(self, dtype):
        return [("recurrent", None)]
