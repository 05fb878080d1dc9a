"""Feed-forward parts."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import FeedForward, Product, StepContext
from .registry import register_feed_forward
from .spec import ParamSpec, PartSpec


@register_feed_forward("swiglu")
class SwiGLU(FeedForward):
    """down(silu(gate(x)) * up(x)), no biases (mini_hisparse/model.py:63-71).

    gate_proj and up_proj are stacked into one [2 I, H] weight at load, in the layout the
    runtime's product wants (interleaved in blocks when the gate is fused into the product's
    epilogue); the checkpoint names stay gate_proj / up_proj / down_proj.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.gate_block = self.inter
        self.down = None

    def parameters(self):
        return {
            "gate_proj.weight": ParamSpec((self.inter, self.hidden)),
            "up_proj.weight": ParamSpec((self.inter, self.hidden)),
            "down_proj.weight": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors):
        self.gate_up, self.gate_block = self.rt.swiglu_layout(tensors["gate_proj.weight"], tensors["up_proj.weight"])
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws = ctx.rt, ctx.ws
        act = rt.linear_swiglu(h, self.gate_up, self.gate_block, ws, "ff_act")
        return rt.linear(act, self.down, ws, "ff_out")
