"""Make the golden outputs: run KiritoHugh/mini-hisparse's OWN model code on a tiny random model.

    python tests/golden/make_golden.py --reference /path/to/mini-hisparse

The reference's ``MiniModel`` (mini_hisparse/model.py:91-181) imports and runs on the CPU.  This
script draws float32 weights from a fixed seed, loads them into ``MiniModel`` with
``load_state_dict(strict=True)`` (its tensor names are Hugging Face's), and records
  * the logits of ``MiniModel.prefill(tokens[:i+1])`` for every prefix (the reference returns
    the last position only, model.py:181), and
  * the greedy tokens of the reference's ``Engine.run()`` (mini_hisparse/engine.py:131-135) over
    its page-cache reference (reference/cache.py), prefill once and then decode.
It writes the model as a folder (config.json, model.safetensors) and the outputs beside it in
``tests/golden/tiny_ref/``.  ``tests/test_plain.py`` compares the plain implementation with
these files; nothing here is imported by the tests.
"""
import argparse
import json
import sys
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
sys.path.insert(0, str(HERE.parent.parent))

CONFIG = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=96, hidden_size=48,
    intermediate_size=80, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=2,
    rms_norm_eps=1e-5, rope_theta=5000.0, tie_word_embeddings=False, max_position_embeddings=128,
)
TOKENS = 40
NEW_TOKENS = 12


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="a checkout of KiritoHugh/mini-hisparse")
    args = ap.parse_args()
    sys.path.insert(0, args.reference)
    from mini_hisparse.engine import Engine
    from mini_hisparse.model import MiniModel, ModelConfig
    from reference.cache import PagedConfig, PagedKVCache

    from mini_hisparse_b200.weights.safetensors_io import write_safetensors

    torch.manual_seed(20240607)
    torch.set_num_threads(1)
    cfg = ModelConfig(
        vocab_size=CONFIG["vocab_size"], hidden_size=CONFIG["hidden_size"],
        intermediate_size=CONFIG["intermediate_size"], num_hidden_layers=CONFIG["num_hidden_layers"],
        num_attention_heads=CONFIG["num_attention_heads"],
        num_key_value_heads=CONFIG["num_key_value_heads"], rms_norm_eps=CONFIG["rms_norm_eps"],
        rope_theta=CONFIG["rope_theta"],
    )
    model = MiniModel(cfg).eval()
    state = {}
    for name, t in model.state_dict().items():
        if name.endswith("layernorm.weight") or name == "model.norm.weight":
            state[name] = 1.0 + 0.1 * torch.randn(t.shape)
        else:
            state[name] = 0.15 * torch.randn(t.shape)
    model.load_state_dict(state, strict=True)
    tokens = torch.randint(0, cfg.vocab_size, (TOKENS,)).tolist()
    rows = [model.prefill(tokens[: i + 1]) for i in range(TOKENS)]
    logits = torch.stack(rows).float().numpy()

    cache = PagedKVCache(PagedConfig(gpu_pages=64, host_pages=64, page_size=4,
                                     kv_heads=cfg.num_key_value_heads, head_dim=cfg.head_dim, device="cpu"))
    engine = Engine(model, cache)
    engine.add_request("a", tokens[:17], NEW_TOKENS)
    engine.add_request("b", tokens[5:40], NEW_TOKENS)
    generated = engine.run()

    out = HERE / "tiny_ref"
    out.mkdir(exist_ok=True)
    (out / "config.json").write_text(json.dumps(CONFIG, indent=2) + "\n")
    write_safetensors(out / "model.safetensors", {k: v.float() for k, v in state.items()})
    logits.astype("<f4").tofile(out / "prefix_logits.f32")
    (out / "golden.json").write_text(json.dumps({
        "tokens": tokens,
        "logits_shape": list(logits.shape),
        "prompts": {"a": tokens[:17], "b": tokens[5:40]},
        "greedy": generated,
        "made_by": "tests/golden/make_golden.py with mini_hisparse.model.MiniModel on the CPU, float32",
    }, indent=2) + "\n")
    print("wrote", out, "logits", logits.shape, "greedy", generated)


if __name__ == "__main__":
    main()
