"""Dynamic Tanh norm: y = tanh(alpha * x) * w + b with a scalar alpha, a weight and a bias per
channel.  It takes no mean and no variance, so a row's elements do not meet: nothing is reduced."""
from __future__ import annotations

from .. import ops
from .base import Norm, ParamDecl, register_part


@register_part("norm", "dyt")
class DynamicTanh(Norm):
    def __init__(self, *, dtype: str, size: int):
        super().__init__()
        self.size, self.dtype = int(size), dtype
        self.decls = {"weight": ParamDecl((self.size,), role="vector", init=("uniform", 0.5, 1.5)),
                      "bias": ParamDecl((self.size,), role="vector", init=("normal", 0.05)),
                      "alpha": ParamDecl((), role="vector", init=("const", 0.75))}
        self.alpha = 1.0

    def prepare(self):
        self.alpha = float(self.w["alpha"])          # a launch argument: read once, at load

    def forward(self, x, out_dtype, rows=None):
        return ops.dyt_norm(x, self.w["weight"], self.w["bias"], self.alpha, out_dtype, rows=rows)

    def kernel_modules(self, dtype):
        return [("elementwise", None)]
