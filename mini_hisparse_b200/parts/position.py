"""Position encodings.  A mixer holds one and hands its constants to its kernels."""
from __future__ import annotations

import torch

from .base import Part
from .registry import register_position
from .spec import PartSpec


class Position(Part):
    """What a mixer's kernels ask of a position encoding that turns pairs of q and k elements.

    ``rotary_dim``: how many leading elements of a head are rotated (0: none); ``inv_freq``: the
    float32 frequencies [rotary_dim / 2] on the device, the kernels form
    ``angle = float(position) * inv_freq[i]``; ``interleaved``: angle i turns the pair
    (2i, 2i + 1) instead of (i, i + rotary_dim / 2).  An encoding of another kind (a bias on the
    scores, a learned table) is a part of its own that its mixer knows how to use.
    """

    rotary_dim = 0
    inv_freq = None
    interleaved = False

    @property
    def rotates(self) -> bool:
        return self.rotary_dim > 0


@register_position("rotary")
class Rotary(Position):
    """Rotary encoding.  The reference's form (mini_hisparse/model.py:141-151) is the default:
    half-split pairs over the whole head, inv_freq[i] = theta ** (-(2 i) / head_dim), i < head_dim / 2,
    computed in float32 exactly as the reference does (``theta ** (-arange(0, d, 2).float() / d)``).

    Parameters: head_dim, theta; optional ``rotary_dim`` (rotate only the first rotary_dim elements
    of a head, frequencies theta ** (-(2 i) / rotary_dim)) and ``style`` ("half_split" pairs
    (i, i + rotary_dim / 2), or "interleaved" pairs (2i, 2i + 1)).
    """

    STYLES = ("half_split", "interleaved")

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.head_dim = int(spec["head_dim"])
        self.theta = float(spec["theta"])
        self.rotary_dim = int(spec.get("rotary_dim") or self.head_dim)
        style = spec.get("style", "half_split")
        if style not in self.STYLES:
            raise ValueError(f"rotary style {style!r} is not one of {self.STYLES}")
        self.interleaved = style == "interleaved"
        if self.rotary_dim % 2 or not 0 < self.rotary_dim <= self.head_dim:
            raise ValueError(f"rotary encoding needs an even rotary_dim of at most head_dim "
                             f"({self.head_dim}), got {self.rotary_dim}")
        inv = self.theta ** (-torch.arange(0, self.rotary_dim, 2).float() / self.rotary_dim)
        self.inv_freq = inv.to(rt.device) if rt is not None else inv


@register_position("none")
class NoPosition(Position):
    """No position encoding: q and k pass unrotated."""
