"""Weights by tensor name: from a model folder's safetensors, or drawn at random from a seed.

The reference adopts a library's modules as weight containers and so inherits their names
(mini_hisparse/model.py:98-125); its test proves the names equal Hugging Face's
(tests/test_engine.py:94, strict load).  Here the model lists the tensors it expects
(name, shape, role) and the loader reads exactly those, reporting every problem at once.

Dtypes on the device: "matrix" tensors take the compute dtype (bfloat16 for serving, float32
on the 32-bit path); "vector" tensors (norm weights, biases) are held in float32 whatever the
file stores, so a tensor stored in 32-bit stays so; "table" tensors are int32.
"""
from __future__ import annotations

import hashlib
import json
from pathlib import Path

import torch

from .safetensors_io import Checkpoint, write_safetensors


class WeightError(ValueError):
    """The checkpoint does not fit the model; the message lists every mismatch."""


def _target_dtype(role: str, compute_dtype: torch.dtype) -> torch.dtype:
    if role == "vector":
        return torch.float32
    if role == "table":
        return torch.int32
    return compute_dtype


def check_names(expected: dict, available: dict[str, tuple]) -> None:
    """Raise one WeightError naming missing tensors, unexpected tensors and wrong shapes."""
    missing = [n for n, ps in expected.items() if n not in available and not ps.optional]
    unexpected = [n for n in available if n not in expected]
    wrong = [
        f"{n}: file has {list(available[n])}, model wants {list(ps.shape)}"
        for n, ps in expected.items()
        if n in available and tuple(available[n]) != tuple(ps.shape)
    ]
    if missing or unexpected or wrong:
        lines = ["the checkpoint does not match the model:"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(sorted(missing)))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(sorted(unexpected)))
        if wrong:
            lines.append(f"  wrong shape ({len(wrong)}): " + "; ".join(sorted(wrong)))
        raise WeightError("\n".join(lines))


def _deliver(model, fetch) -> None:
    """Hand every part its tensors (fetched by full name) and let it re-lay them out."""
    rt = model.rt
    for prefix, part in model.named_parts():
        tensors = {}
        for local, ps in part.parameters().items():
            t = fetch(f"{prefix}.{local}", ps)
            if t is not None:
                tensors[local] = t.to(device=rt.device, dtype=_target_dtype(ps.role, rt.dtype))
        part.load(tensors)
    model.finish_loading()


def load_weights(model, folder) -> None:
    ckpt = Checkpoint(folder)
    try:
        expected = model.expected_tensors()
        check_names(expected, {n: ckpt.info(n).shape for n in ckpt.names()})

        def fetch(name, ps):
            return ckpt.read(name) if name in ckpt.tensors else None

        _deliver(model, fetch)
    finally:
        ckpt.close()


# ---- random weights -----------------------------------------------------------------------------
def _tensor_seed(seed: int, name: str) -> int:
    h = hashlib.sha256(f"{seed}:{name}".encode()).digest()
    return int.from_bytes(h[:8], "little") & ((1 << 63) - 1)


def draw(name: str, ps, seed: int, device="cpu", matrix_std: float | None = None) -> torch.Tensor:
    """One tensor of the random-weights mode: its own generator, seeded by (seed, name), so the
    values do not depend on the order in which tensors are drawn.  float32 values."""
    kind, mean, std = ps.init
    if matrix_std is not None and ps.role == "matrix":
        std = matrix_std
    if kind != "normal":
        raise ValueError(f"unknown init {ps.init!r} for {name}")
    gen = torch.Generator(device=device)
    gen.manual_seed(_tensor_seed(seed, name))
    t = torch.empty(ps.shape, dtype=torch.float32, device=device)
    t.normal_(mean, std, generator=gen)
    return t


def init_random(model, seed: int) -> None:
    """Fill the model with seeded random weights drawn on its device (large shapes, no file)."""
    rt = model.rt

    def fetch(name, ps):
        if ps.optional:
            return None
        return draw(name, ps, seed, device=rt.device)

    _deliver(model, fetch)


def write_random_model(config: dict, seed: int, folder, dtype: torch.dtype = torch.bfloat16,
                       matrix_std: float | None = None) -> Path:
    """Write a model folder (config.json, model.safetensors) for a configuration and a seed.

    Weights and biases are normal(0, 0.02), norm weights 1 + normal(0, 0.1); matrices are stored
    in ``dtype``, vectors in float32.  ``matrix_std`` replaces the 0.02 of the matrices (tests use
    a larger one, so that attention is not near-uniform and a wrong key shows).
    """
    from ..config.registry import resolve
    from ..parts.spec import ParamSpec  # noqa: F401  (documents what expected_tensors returns)
    from .expected import expected_tensors_of_spec

    folder = Path(folder)
    folder.mkdir(parents=True, exist_ok=True)
    _, spec = resolve(config)
    tensors = {}
    for name, ps in expected_tensors_of_spec(spec).items():
        if ps.optional:
            continue
        t = draw(name, ps, seed, matrix_std=matrix_std)
        tensors[name] = t.to(_target_dtype(ps.role, dtype))
    (folder / "config.json").write_text(json.dumps(config, indent=2) + "\n")
    write_safetensors(folder / "model.safetensors", tensors, metadata={"format": "pt", "seed": str(seed)})
    return folder
