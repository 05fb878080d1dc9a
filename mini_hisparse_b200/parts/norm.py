"""RMSNorm: width and eps are parameters of the part (mini_hisparse/model.py:43-51)."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Norm, Product, StepContext
from .registry import register_norm
from .spec import ParamSpec, PartSpec


@register_norm("rmsnorm")
class RMSNorm(Norm):
    """y = x * rsqrt(mean(x^2) + eps) * weight, computed in float32 from the float32 residual.

    The weight is a plain multiplier (not 1 + w) and there is no bias, as in the reference.
    With ``delta`` the kernel first adds it to the residual (and writes the sum back when all
    rows are processed), so the residual add costs no extra pass over memory.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.width = int(spec["width"])
        self.eps = float(spec["eps"])
        self.weight = None

    def parameters(self):
        return {"weight": ParamSpec((self.width,), role="vector", init=("normal", 1.0, 0.1))}

    def load(self, tensors):
        self.weight = tensors["weight"]

    def forward(self, x, ctx: StepContext, delta: Product | None = None, rows=None, name="h"):
        R = x.shape[0] if rows is None else rows.shape[0]
        out = ctx.ws.get(name, (R, self.width), ctx.rt.dtype)
        if delta is None:
            K.add_rmsnorm(x, self.weight, self.eps, out, rows=rows)
        else:
            K.add_rmsnorm(x, self.weight, self.eps, out, delta=delta.tensor, nsplit=delta.nsplit,
                          split_stride=delta.split_stride, rows=rows)
        return out
