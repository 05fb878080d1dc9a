"""The tensors a ModelSpec expects, without a device: parts are built with no runtime."""
from __future__ import annotations

from ..parts.registry import BLOCKS, EMBEDDINGS, HEADS, NORMS
from ..parts.spec import ModelSpec, ParamSpec


def expected_tensors_of_spec(spec: ModelSpec) -> dict[str, ParamSpec]:
    out: dict[str, ParamSpec] = {}

    def add(prefix, part):
        for local, ps in part.parameters().items():
            out[f"{prefix}.{local}"] = ps

    add(spec.embedding_name, EMBEDDINGS.build(spec.embedding, rt=None))
    for layer in spec.layers:
        block = BLOCKS.get(layer.block)(layer, None)
        for role, part in block.parts().items():
            add(f"{layer.prefix}.{layer.name_of(role)}", part)
    add(spec.final_norm_name, NORMS.build(spec.final_norm, rt=None))
    add(spec.head_name, HEADS.build(spec.head, rt=None))
    return out
