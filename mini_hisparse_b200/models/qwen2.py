"""Qwen2 dense decoder as data: the ModelSpec of a Qwen2Config and its registry entry.

Every layer is the same pre-norm block (mini_hisparse/model.py:74-88): RMSNorm, grouped-query
attention with q/k/v bias and half-split rotary positions, RMSNorm, SwiGLU.  Tensor names are
Hugging Face's (model.embed_tokens, model.layers.N.{input_layernorm,self_attn,
post_attention_layernorm,mlp}, model.norm, lm_head), which the reference's module tree equals.
"""
from __future__ import annotations

from ..config.qwen2 import Qwen2Config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def qwen2_spec(cfg: Qwen2Config) -> ModelSpec:
    norm = PartSpec.make("rmsnorm", width=cfg.hidden_size, eps=cfg.rms_norm_eps)
    position = PartSpec.make("rotary", head_dim=cfg.head_dim, theta=cfg.rope_theta)
    mixer = PartSpec.make(
        "gq_attention",
        hidden_size=cfg.hidden_size,
        q_heads=cfg.num_attention_heads,
        kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim,
        qkv_bias=True,
        window=None,
        position=position,
    )
    ff = PartSpec.make("swiglu", hidden_size=cfg.hidden_size, intermediate_size=cfg.intermediate_size)
    layers = tuple(
        LayerSpec.pre_norm(f"model.layers.{i}", mixer=mixer, mixer_norm=norm, feed_forward=ff, ff_norm=norm)
        for i in range(cfg.num_hidden_layers)
    )
    return ModelSpec(
        architecture="Qwen2ForCausalLM",
        vocab_size=cfg.vocab_size,
        hidden_size=cfg.hidden_size,
        embedding=PartSpec.make("token_embedding", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size),
        embedding_name="model.embed_tokens",
        layers=layers,
        order=tuple(RunEntry(i) for i in range(cfg.num_hidden_layers)),
        final_norm=norm,
        final_norm_name="model.norm",
        head=PartSpec.make("lm_head", vocab_size=cfg.vocab_size, hidden_size=cfg.hidden_size,
                           tied=cfg.tie_word_embeddings),
        head_name="lm_head",
        max_positions=cfg.max_position_embeddings,
        eos_token_id=cfg.eos_token_id,
    )


register_architecture("Qwen2ForCausalLM", Qwen2Config, qwen2_spec, replace=True)
