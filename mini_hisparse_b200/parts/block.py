"""Block arrangements: how a layer's norms, mixer and feed-forward are wired to the residual."""
from __future__ import annotations

from .base import Block, CacheView, Product, StepContext
from .registry import FEED_FORWARDS, MIXERS, NORMS, register_block
from .spec import LayerSpec


@register_block("pre_norm")
class PreNormBlock(Block):
    """x = x + mixer(norm1(x)); x = x + ff(norm2(x))   (mini_hisparse/model.py:137,155-158).

    The residual adds are folded into the norms that follow them: the block receives the
    previous block's still-unadded output as ``pending`` and returns its own.
    """

    def __init__(self, spec: LayerSpec, rt):
        self.spec = spec
        self.mixer_norm = NORMS.build(spec.part("mixer_norm"), rt=rt)
        self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
        self.ff_norm = NORMS.build(spec.part("ff_norm"), rt=rt)
        self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt)

    def parts(self):
        return {
            "mixer_norm": self.mixer_norm,
            "mixer": self.mixer,
            "ff_norm": self.ff_norm,
            "feed_forward": self.feed_forward,
        }

    def forward(self, x, pending: Product | None, ctx: StepContext, cache: CacheView | None) -> Product:
        h = self.mixer_norm.forward(x, ctx, delta=pending)
        a = self.mixer.forward(h, ctx, cache)
        h = self.ff_norm.forward(x, ctx, delta=a)
        return self.feed_forward.forward(h, ctx)
