"""Token embedding and output head."""
from __future__ import annotations

import torch

from ..kernels import api as K
from .base import Part, Product, StepContext
from .registry import EMBEDDINGS, HEADS
from .spec import ParamSpec, PartSpec


@EMBEDDINGS.register("token_embedding")
class TokenEmbedding(Part):
    """x = table[tokens], no scaling (mini_hisparse/model.py:86,166); output is the float32 residual."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.vocab = int(spec["vocab_size"])
        self.width = int(spec["hidden_size"])
        self.weight = None

    def parameters(self):
        return {"weight": ParamSpec((self.vocab, self.width))}

    def load(self, tensors):
        self.weight = tensors["weight"].contiguous()

    def forward(self, ctx: StepContext) -> torch.Tensor:
        x = ctx.ws.get("residual", (ctx.T, self.width), torch.float32)
        K.embed(self.weight, ctx.tokens, x, status=ctx.status)
        return x


@HEADS.register("lm_head")
class LMHead(Part):
    """logits = h W^T in float32, no bias (mini_hisparse/model.py:96,181).  With ``tied`` the
    embedding table is the weight and the checkpoint holds no lm_head tensor."""

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.vocab = int(spec["vocab_size"])
        self.width = int(spec["hidden_size"])
        self.tied = bool(spec["tied"])
        self.weight = None

    def parameters(self):
        if self.tied:
            return {"weight": ParamSpec((self.vocab, self.width), optional=True)}
        return {"weight": ParamSpec((self.vocab, self.width))}

    def load(self, tensors):
        if not self.tied:
            self.weight = tensors["weight"].contiguous()

    def tie(self, embedding: TokenEmbedding):
        self.weight = embedding.weight

    def forward(self, h: torch.Tensor, ctx: StepContext) -> torch.Tensor:
        return ctx.rt.linear(h, self.weight, ctx.ws, "logits", out_dtype=torch.float32,
                             allow_split=False).matrix
