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

    gate_proj and up_proj are stacked into one [2 I, H] weight at load so that one product
    feeds the gate kernel; the checkpoint names stay gate_proj / up_proj / down_proj.
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.inter = int(spec["intermediate_size"])
        self.gate_up = None
        self.down = None

    def parameters(self):
        return {
            "gate_proj.weight": ParamSpec((self.inter, self.hidden)),
            "up_proj.weight": ParamSpec((self.inter, self.hidden)),
            "down_proj.weight": ParamSpec((self.hidden, self.inter)),
        }

    def load(self, tensors):
        self.gate_up = torch.cat((tensors["gate_proj.weight"], tensors["up_proj.weight"]), 0).contiguous()
        self.down = tensors["down_proj.weight"].contiguous()

    def forward(self, h, ctx: StepContext) -> Product:
        rt, ws = ctx.rt, ctx.ws
        gu = rt.linear(h, self.gate_up, ws, "gate_up")
        act = ws.get("ff_act", (h.shape[0], self.inter), rt.dtype)
        K.swiglu(gu.tensor, act, nsplit=gu.nsplit, split_stride=gu.split_stride)
        return rt.linear(act, self.down, ws, "ff_out")
