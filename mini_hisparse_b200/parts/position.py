"""Position encodings.  A mixer holds one and hands its constants to its kernels."""
from __future__ import annotations

import torch

from .base import Part
from .registry import register_position
from .spec import PartSpec


@register_position("rotary")
class Rotary(Part):
    """Half-split rotary encoding (mini_hisparse/model.py:141-151).

    inv_freq[i] = theta ** (-(2 i) / head_dim), i < head_dim / 2, computed in float32 exactly as
    the reference does (``theta ** (-arange(0, d, 2).float() / d)``); the kernel forms
    angle = float(position) * inv_freq[i] and rotates the pair (j, j + d/2).
    """

    rotates = True

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.head_dim = int(spec["head_dim"])
        self.theta = float(spec["theta"])
        if self.head_dim % 2:
            raise ValueError(f"rotary encoding needs an even head_dim, got {self.head_dim}")
        inv = self.theta ** (-torch.arange(0, self.head_dim, 2).float() / self.head_dim)
        self.inv_freq = inv.to(rt.device) if rt is not None else inv


@register_position("none")
class NoPosition(Part):
    """No position encoding: q and k pass unrotated."""

    rotates = False

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.inv_freq = None
