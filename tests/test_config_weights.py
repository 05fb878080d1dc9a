"""Configuration, registry, safetensors, loader errors.  No GPU."""
import json

import pytest
import torch

from conftest import TINY_A, TINY_B, TINY_C
from mini_hisparse_b200 import ConfigError, Qwen2Config, WeightError, known_architectures, resolve, write_random_model
from mini_hisparse_b200.config.registry import architecture_of
from mini_hisparse_b200.weights import Checkpoint, check_names, write_safetensors
from mini_hisparse_b200.weights.expected import expected_tensors_of_spec
from plain import qwen2_plain as P


def test_config_reads_its_own_keys():
    a = Qwen2Config.from_dict(TINY_A)
    assert (a.hidden_size, a.num_attention_heads, a.num_key_value_heads, a.head_dim) == (64, 4, 2, 16)
    assert a.tie_word_embeddings and a.rope_theta == 10000.0 and a.rms_norm_eps == 1e-6
    c = Qwen2Config.from_dict(TINY_C)
    assert c.head_dim == 48 and c.rope_theta == 50000.0      # rope_parameters form, explicit head_dim
    assert Qwen2Config.from_dict(a.to_dict()) == a


@pytest.mark.parametrize("key", ["vocab_size", "hidden_size", "intermediate_size", "num_hidden_layers",
                                 "num_attention_heads", "rms_norm_eps", "rope_theta"])
def test_no_size_has_a_default(key):
    d = dict(TINY_A)
    del d[key]
    with pytest.raises(ConfigError, match=key):
        Qwen2Config.from_dict(d)


@pytest.mark.parametrize("patch,word", [
    (dict(use_sliding_window=True), "sliding"),
    (dict(hidden_act="gelu"), "gelu"),
    (dict(rope_scaling={"type": "yarn", "factor": 4.0}), "yarn"),
    (dict(num_key_value_heads=3), "multiple"),
    (dict(head_dim=15), "even"),
    (dict(model_type="llama"), "llama"),
])
def test_unsupported_options_are_refused(patch, word):
    with pytest.raises(ConfigError, match=word):
        Qwen2Config.from_dict({**TINY_A, **patch})


def test_registry_names_the_model():
    assert "Qwen2ForCausalLM" in known_architectures()
    cfg, spec = resolve(TINY_B)
    assert spec.architecture == "Qwen2ForCausalLM" and len(spec.layers) == 3 and len(spec.order) == 3
    assert spec.layers[0].part("mixer")["q_heads"] == 3 and spec.layers[0].part("mixer")["kv_heads"] == 1
    with pytest.raises(KeyError, match="Qwen2ForCausalLM"):
        architecture_of({"architectures": ["MysteryForCausalLM"]})


def test_safetensors_round_trip_and_plain_reader(tmp_path):
    t = {"a": torch.randn(3, 5), "b": torch.randn(7).bfloat16(), "c": torch.arange(6, dtype=torch.int32).view(2, 3)}
    write_safetensors(tmp_path / "model.safetensors", t)
    ck = Checkpoint(tmp_path)
    assert set(ck.names()) == set(t)
    for k, v in t.items():
        assert ck.info(k).shape == tuple(v.shape) and ck.info(k).dtype == v.dtype
        assert torch.equal(ck.read(k), v)
    other = P.read_safetensors(tmp_path / "model.safetensors")    # the oracle's own reader
    for k, v in t.items():
        assert torch.equal(other[k], v)


def test_random_model_folder(tmp_path):
    write_random_model(TINY_A, 3, tmp_path / "m", dtype=torch.bfloat16)
    write_random_model(TINY_A, 3, tmp_path / "n", dtype=torch.bfloat16)
    write_random_model(TINY_A, 4, tmp_path / "o", dtype=torch.bfloat16)
    a, b, c = (P.read_safetensors(tmp_path / x / "model.safetensors") for x in "mno")
    assert json.loads((tmp_path / "m" / "config.json").read_text())["hidden_size"] == 64
    assert set(a) == set(expected_tensors_of_spec(resolve(TINY_A)[1])) - {"lm_head.weight"}
    assert all(torch.equal(a[k], b[k]) for k in a) and not torch.equal(a["model.norm.weight"], c["model.norm.weight"])
    w = a["model.layers.0.mlp.up_proj.weight"]
    assert w.dtype == torch.bfloat16 and abs(float(w.float().std()) - 0.02) < 0.002
    n = a["model.layers.1.input_layernorm.weight"]
    assert n.dtype == torch.float32 and abs(float(n.mean()) - 1.0) < 0.05


def test_one_error_lists_everything(tmp_path):
    _, spec = resolve(TINY_B)
    expected = expected_tensors_of_spec(spec)
    have = {n: ps.shape for n, ps in expected.items()}
    del have["model.norm.weight"], have["model.layers.1.self_attn.k_proj.bias"]
    have["model.layers.0.mlp.down_proj.weight"] = (5, 5)
    have["model.layers.9.extra.weight"] = (1,)
    with pytest.raises(WeightError) as e:
        check_names(expected, have)
    msg = str(e.value)
    assert "missing (2)" in msg and "model.norm.weight" in msg and "k_proj.bias" in msg
    assert "unexpected (1)" in msg and "model.layers.9.extra.weight" in msg
    assert "wrong shape (1)" in msg and "[5, 5]" in msg and "[96, 256]" in msg


def test_tied_head_needs_no_lm_head_tensor():
    exp_a = expected_tensors_of_spec(resolve(TINY_A)[1])
    exp_b = expected_tensors_of_spec(resolve(TINY_B)[1])
    assert exp_a["lm_head.weight"].optional and not exp_b["lm_head.weight"].optional
    have = {n: ps.shape for n, ps in exp_a.items() if n != "lm_head.weight"}
    check_names(exp_a, have)


def test_sharded_model_folder(tmp_path):
    """A folder of two shards and model.safetensors.index.json (how large checkpoints come) is read
    like a single file: names and shapes are checked over all shards, and a tensor the index
    promises but no shard holds is reported as missing."""
    write_random_model(TINY_B, 5, tmp_path / "one", dtype=torch.bfloat16)
    tensors = P.read_safetensors(tmp_path / "one" / "model.safetensors")
    names = sorted(tensors)
    halves = [names[: len(names) // 2], names[len(names) // 2:]]
    folder = tmp_path / "sharded"
    folder.mkdir()
    weight_map = {}
    for i, part in enumerate(halves):
        fname = f"model-{i + 1:05d}-of-00002.safetensors"
        write_safetensors(folder / fname, {n: tensors[n] for n in part})
        weight_map.update({n: fname for n in part})
    (folder / "config.json").write_text((tmp_path / "one" / "config.json").read_text())
    (folder / "model.safetensors.index.json").write_text(json.dumps({"metadata": {}, "weight_map": weight_map}))
    ck = Checkpoint(folder)
    assert len(ck.files) == 2 and set(ck.names()) == set(names)
    for n in (names[0], names[-1]):
        assert torch.equal(ck.read(n), tensors[n])
    expected = expected_tensors_of_spec(resolve(TINY_B)[1])
    check_names(expected, {n: ck.info(n).shape for n in ck.names()})
    ck.close()
    # drop a tensor from the second shard: one error names it
    victim = halves[1][0]
    write_safetensors(folder / "model-00002-of-00002.safetensors", {n: tensors[n] for n in halves[1][1:]})
    ck = Checkpoint(folder)
    with pytest.raises(WeightError, match=victim.replace(".", r"\.")):
        check_names(expected, {n: ck.info(n).shape for n in ck.names()})
    ck.close()
