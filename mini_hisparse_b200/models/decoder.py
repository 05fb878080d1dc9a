"""A decoder built from a ModelSpec: embedding, blocks in run order, final norm, output head.

The model knows nothing about requests or pages; it runs the tokens of one StepContext and
returns float32 logits at the wanted rows.  The order of the reference's forward
(mini_hisparse/model.py:160-181, 183-226) is kept: embed, then per layer norm -> mixer (which
appends to the cache before it attends) -> residual -> norm -> feed-forward -> residual, then
the final norm and the head on the wanted rows only.
"""
from __future__ import annotations

import torch

from ..kernels import api as K
from ..parts.base import CacheView, Product, Runtime, StepContext
from ..parts.registry import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..parts.spec import ModelSpec, ParamSpec


class DecoderModel:
    def __init__(self, spec: ModelSpec, rt: Runtime, config=None):
        self.spec, self.rt, self.config = spec, rt, config
        self.embedding = EMBEDDINGS.build(spec.embedding, rt=rt)
        self.blocks = [BLOCKS.get(layer.block)(layer, rt) for layer in spec.layers]
        self.final_norm = NORMS.build(spec.final_norm, rt=rt)
        self.head = HEADS.build(spec.head, rt=rt)
        # cache entries: one per run entry that owns a cache
        self.entry_cache: list[int] = []      # run entry -> cache entry index
        self.cache_needs = []
        for i, e in enumerate(spec.order):
            if e.cache_of is None:
                self.entry_cache.append(len(self.cache_needs))
                self.cache_needs.append(self.blocks[e.layer].cache_need())
            else:
                owner = self.entry_cache[e.cache_of]
                mine, theirs = self.blocks[e.layer].cache_need(), self.cache_needs[owner]
                if mine != theirs:
                    raise ValueError(
                        f"run entry {i} reads the cache of entry {e.cache_of}, but their needs differ: "
                        f"{mine} vs {theirs}"
                    )
                self.entry_cache.append(owner)
        self.loaded = False

    # ---- parameters --------------------------------------------------------------------------
    def named_parts(self):
        """(checkpoint prefix, part) for every part that stores tensors."""
        yield self.spec.embedding_name, self.embedding
        for layer, block in zip(self.spec.layers, self.blocks):
            for role, part in block.parts().items():
                yield f"{layer.prefix}.{layer.name_of(role)}", part
        yield self.spec.final_norm_name, self.final_norm
        yield self.spec.head_name, self.head

    def kernel_modules(self) -> tuple[str, ...]:
        """What this model's steps launch: the runtime's libraries and those of its parts."""
        mods = list(self.rt.kernel_modules())
        for _, part in self.named_parts():
            for m in part.kernel_modules():
                if m not in mods:
                    mods.append(m)
        return tuple(mods)

    def expected_tensors(self) -> dict[str, ParamSpec]:
        out = {}
        for prefix, part in self.named_parts():
            for local, ps in part.parameters().items():
                out[f"{prefix}.{local}"] = ps
        return out

    def finish_loading(self):
        if getattr(self.head, "tied", False):
            self.head.tie(self.embedding)
        self.loaded = True

    def weight_bytes(self) -> int:
        seen, total = set(), 0
        parts = [p for _, p in self.named_parts()]
        for part in parts:
            for v in vars(part).values():
                if isinstance(v, torch.Tensor) and v.data_ptr() not in seen:
                    seen.add(v.data_ptr())
                    total += v.numel() * v.element_size()
        return total

    @property
    def graph_safe(self) -> bool:
        return all(b.graph_safe for b in self.blocks)

    # ---- forward --------------------------------------------------------------------------------
    def forward(self, ctx: StepContext, caches: list[CacheView | None], rows: torch.Tensor | None,
                observer=None) -> torch.Tensor | None:
        """Run the batch; return logits [R, V] float32 at ``rows`` (None: no logits wanted).

        ``observer(i, residual, pending)`` is called after every run entry i with the float32
        residual stream [T, H] and the entry's output that is not yet added to it (a Product), and
        once more as ``observer("final", residual, None)`` with everything added: the reference's
        layer hook (mini_hisparse/model.py:171-172, 202-203) for this engine's fused residual adds.
        The tensors are the step's own buffers: copy what is to be kept."""
        if not self.loaded:
            raise RuntimeError("the model has no weights yet")
        x = self.embedding.forward(ctx)
        pending: Product | None = None
        for i, entry in enumerate(self.spec.order):
            view = caches[i]
            pending = self.blocks[entry.layer].forward(x, pending, ctx, view)
            if observer is not None:
                observer(i, x, pending)
        if observer is not None and pending is not None:
            # the hook's last call sees the finished residual stream (the head needs only its wanted
            # rows and never adds the last output into every row)
            K.residual_add(x, pending.tensor, nsplit=pending.nsplit, split_stride=pending.split_stride)
            observer("final", x, None)
            pending = None
        if rows is None or rows.numel() == 0:
            return None
        h = self.final_norm.forward(x, ctx, delta=pending, rows=rows, name="h_rows")
        return self.head.forward(h, ctx)
