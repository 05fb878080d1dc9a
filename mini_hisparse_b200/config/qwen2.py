"""Typed Qwen2 configuration, read from the keys of the architecture's own config.json.

The reference keeps eight sizes in a dataclass and derives ``head_dim`` from
``hidden_size // num_attention_heads`` (mini_hisparse/model.py:19-40); when it loads
a checkpoint it copies those fields by name from the Hugging Face config and rejects
non-default RoPE, sliding windows and activations other than SiLU
(mini_hisparse/model.py:103-123).  This class reads the same keys straight from
``config.json``; no size has a default here.
"""
from __future__ import annotations

import json
from dataclasses import dataclass, field, asdict
from pathlib import Path
from typing import Any, Mapping


class ConfigError(ValueError):
    """config.json is missing a key, or asks for something this architecture cannot do."""


_REQUIRED = (
    "vocab_size",
    "hidden_size",
    "intermediate_size",
    "num_hidden_layers",
    "num_attention_heads",
    "rms_norm_eps",
)


@dataclass(frozen=True)
class Qwen2Config:
    vocab_size: int
    hidden_size: int
    intermediate_size: int
    num_hidden_layers: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int | None
    eos_token_id: int | None
    bos_token_id: int | None
    torch_dtype: str | None
    architectures: tuple[str, ...] = field(default=("Qwen2ForCausalLM",))
    model_type: str = "qwen2"

    # ------------------------------------------------------------------
    @classmethod
    def from_dict(cls, d: Mapping[str, Any]) -> "Qwen2Config":
        missing = [k for k in _REQUIRED if k not in d]
        # Transformers 5 moves rope_theta into rope_parameters; older files keep it at the top
        # and put a type into rope_scaling (mini_hisparse/model.py:103-106).
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        theta = rope.get("rope_theta", d.get("rope_theta"))
        if theta is None:
            missing.append("rope_theta")
        if missing:
            raise ConfigError(f"config.json lacks required key(s): {', '.join(missing)}")
        rope_type = rope.get("rope_type", rope.get("type", "default"))
        if rope_type != "default":
            raise ConfigError(
                f"rope type {rope_type!r} is not supported: only Qwen2/Qwen2.5 with standard RoPE"
            )
        if d.get("use_sliding_window", False):
            raise ConfigError("use_sliding_window=true is not supported by the Qwen2 dense engine")
        act = d.get("hidden_act", "silu")
        if act != "silu":
            raise ConfigError(f"hidden_act {act!r} is not supported: Qwen2 uses silu (SwiGLU)")
        model_type = d.get("model_type", "qwen2")
        if model_type != "qwen2":
            raise ConfigError(f"model_type {model_type!r} is not qwen2")
        nq = int(d["num_attention_heads"])
        nkv = int(d.get("num_key_value_heads") or nq)
        hidden = int(d["hidden_size"])
        head_dim = d.get("head_dim")
        if head_dim is None:
            if hidden % nq:
                raise ConfigError(
                    f"hidden_size {hidden} is not divisible by num_attention_heads {nq}"
                )
            head_dim = hidden // nq
        eos = d.get("eos_token_id")
        if isinstance(eos, (list, tuple)):
            eos = eos[0] if eos else None
        cfg = cls(
            vocab_size=int(d["vocab_size"]),
            hidden_size=hidden,
            intermediate_size=int(d["intermediate_size"]),
            num_hidden_layers=int(d["num_hidden_layers"]),
            num_attention_heads=nq,
            num_key_value_heads=nkv,
            head_dim=int(head_dim),
            rms_norm_eps=float(d["rms_norm_eps"]),
            rope_theta=float(theta),
            tie_word_embeddings=bool(d.get("tie_word_embeddings", False)),
            max_position_embeddings=(
                int(d["max_position_embeddings"]) if d.get("max_position_embeddings") else None
            ),
            eos_token_id=None if eos is None else int(eos),
            bos_token_id=None if d.get("bos_token_id") is None else int(d["bos_token_id"]),
            torch_dtype=d.get("torch_dtype") or d.get("dtype"),
            architectures=tuple(d.get("architectures") or ("Qwen2ForCausalLM",)),
            model_type=model_type,
        )
        cfg.validate()
        return cfg

    @classmethod
    def from_json(cls, path) -> "Qwen2Config":
        path = Path(path)
        if path.is_dir():
            path = path / "config.json"
        return cls.from_dict(json.loads(path.read_text()))

    # ------------------------------------------------------------------
    def validate(self) -> None:
        """Grouped-query attention and half-split RoPE need these (mini_hisparse/model.py:34-40)."""
        for name in (
            "vocab_size",
            "hidden_size",
            "intermediate_size",
            "num_hidden_layers",
            "num_attention_heads",
            "num_key_value_heads",
            "head_dim",
        ):
            if getattr(self, name) < 1:
                raise ConfigError(f"{name} must be positive, got {getattr(self, name)}")
        if self.num_attention_heads % self.num_key_value_heads:
            raise ConfigError(
                f"num_attention_heads {self.num_attention_heads} is not a multiple of "
                f"num_key_value_heads {self.num_key_value_heads}"
            )
        if self.head_dim % 2:
            raise ConfigError(f"head_dim {self.head_dim} must be even for RoPE")
        if not self.rms_norm_eps > 0:
            raise ConfigError("rms_norm_eps must be positive")
        if not self.rope_theta > 0:
            raise ConfigError("rope_theta must be positive")

    def to_dict(self) -> dict:
        d = asdict(self)
        d["architectures"] = list(self.architectures)
        d["hidden_act"] = "silu"
        d["use_sliding_window"] = False
        return {k: v for k, v in d.items() if v is not None}

    def parameter_count(self) -> int:
        h, i, v = self.hidden_size, self.intermediate_size, self.vocab_size
        q = self.num_attention_heads * self.head_dim
        kv = self.num_key_value_heads * self.head_dim
        layer = h * q + q + 2 * (h * kv + kv) + q * h + 3 * h * i + 2 * h
        head = 0 if self.tie_word_embeddings else v * h
        return v * h + self.num_hidden_layers * layer + h + head
