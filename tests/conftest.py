"""Shared fixtures: the two tiny Qwen2 configurations, model folders with random weights, and a
driver for ``bin/trace_run``.  Model folders live in pytest's temporary folders only."""
from __future__ import annotations

import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

# Two configurations that differ in every size and option (layers, width, heads, groups, head
# size, feed-forward width, vocabulary, rope_theta, eps, tied head, positions, page size).
TINY_A = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=512, hidden_size=64,
    intermediate_size=176, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    rms_norm_eps=1e-6, rope_theta=10000.0, tie_word_embeddings=True, max_position_embeddings=256,
    hidden_act="silu", use_sliding_window=False,
)
TINY_B = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=1000, hidden_size=96,
    intermediate_size=256, num_hidden_layers=3, num_attention_heads=3, num_key_value_heads=1,
    rms_norm_eps=1e-5, rope_theta=1000000.0, tie_word_embeddings=False,
    max_position_embeddings=512, hidden_act="silu", use_sliding_window=False,
)
# A third shape with an explicit head_dim that is not hidden/heads, 48 wide, 5 query heads per
# KV head and a vocabulary that is no multiple of anything.
TINY_C = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=777, hidden_size=80,
    intermediate_size=136, num_hidden_layers=2, num_attention_heads=10, num_key_value_heads=2,
    head_dim=48, rms_norm_eps=3e-6, rope_parameters={"rope_theta": 50000.0, "rope_type": "default"},
    tie_word_embeddings=False, max_position_embeddings=1024,
)
# A fourth shape that no tensor-core kernel takes in bfloat16: a width that is no multiple of 8
# (the CUDA-core product), a head size of 80 (the CUDA-core attention), a feed-forward width that
# is no multiple of 16 (the plain gate/up layout), as many KV heads as query heads, pages of 8.
TINY_D = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=1001, hidden_size=100,
    intermediate_size=150, num_hidden_layers=2, num_attention_heads=5, num_key_value_heads=5,
    head_dim=80, rms_norm_eps=1e-4, rope_theta=12345.6, tie_word_embeddings=True,
    max_position_embeddings=300,
)
# A fifth shape for pages that are no power of two and do not divide the kernels' 64-key tiles: head
# size 64 (in bfloat16 the tensor-core kernels that take any page size), pages of 24 positions.
TINY_E = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=600, hidden_size=128,
    intermediate_size=208, num_hidden_layers=2, num_attention_heads=4, num_key_value_heads=2,
    head_dim=64, rms_norm_eps=2e-6, rope_theta=20000.0, tie_word_embeddings=False,
    max_position_embeddings=400,
)
# A sixth: head size 48 (the CUDA-core attention in both dtypes) over pages of 7 positions.
TINY_F = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=333, hidden_size=72,
    intermediate_size=112, num_hidden_layers=2, num_attention_heads=6, num_key_value_heads=3,
    head_dim=48, rms_norm_eps=1e-5, rope_theta=3000.0, tie_word_embeddings=True,
    max_position_embeddings=300,
)
TINY = {"A": (TINY_A, 16), "B": (TINY_B, 32), "C": (TINY_C, 16), "D": (TINY_D, 8), "E": (TINY_E, 24),
        "F": (TINY_F, 7)}


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


def pytest_collection_modifyitems(config, items):
    if torch.cuda.is_available():
        return
    skip = pytest.mark.skip(reason="no CUDA device")
    for item in items:
        if "gpu" in item.keywords:
            item.add_marker(skip)


def random_tokens(vocab: int, n: int, seed: int) -> list[int]:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, vocab, (n,), generator=g).tolist()


def make_folder(tmp_path_factory, name: str, seed: int = 11, matrix_std: float = 0.1) -> Path:
    from mini_hisparse_b200 import write_random_model

    cfg, _ = TINY[name]
    folder = tmp_path_factory.mktemp(f"tiny{name}")
    write_random_model(cfg, seed, folder, dtype=torch.bfloat16, matrix_std=matrix_std)
    return folder


@pytest.fixture(scope="session")
def folders(tmp_path_factory):
    """Model folders of the tiny configurations, bfloat16 matrices (both dtypes read the same values)."""
    return {name: make_folder(tmp_path_factory, name) for name in TINY}


# bfloat16 against float32 (the plain implementation, or the engine's own float32 run), tiny models:
# activations are rounded to 8 bits of mantissa after every part, and with widths of 64 to 128 and
# matrices of standard deviation 0.1 the roundings do not average out.  Two measures per logit row:
# the largest error as a share of the request's largest logit, and the root-mean-square error of
# the row as a share of the row's root mean square.  The bounds are twice the worst that the replay
# tests measured on a B200 over all cuts, shape by shape (A 0.0110 / 0.0138, B 0.0176 / 0.0194,
# C 0.0069 / 0.0087, D 0.0120 / 0.0150, E 0.0164 / 0.0205, F 0.0083 / 0.0104).
BF16_BOUNDS = {"A": (0.022, 0.028), "B": (0.035, 0.039), "C": (0.014, 0.018), "D": (0.024, 0.030),
               "E": (0.033, 0.041), "F": (0.017, 0.021)}


def tolerances(dtype: str, ref: torch.Tensor, name: str) -> dict:
    """float32: rounding of a different summation order.  bfloat16: the measured bound of the
    shape ``name``, relative to the size of the request's logits."""
    if dtype == "float32":
        return dict(atol=3e-5, rtol=3e-5)
    return dict(atol=BF16_BOUNDS[name][0] * float(ref.abs().max()), rtol=0.0)


def row_rms_error(got: torch.Tensor, ref: torch.Tensor) -> float:
    """The worst row's root-mean-square error as a share of that row's root mean square."""
    err = (got.double() - ref.double()).pow(2).mean(-1).sqrt()
    return float((err / ref.double().pow(2).mean(-1).sqrt()).max())


class TraceRun:
    """Drives bin/trace_run over pipes: one JSON line in, ``done <step>`` out, logits from the file."""

    def __init__(self, folder, dtype: str, out_dir, max_tokens: int, page_size: int = 16, extra=()):
        self.out = Path(out_dir)
        self.step_no = 0
        env = dict(os.environ, PYTHONUNBUFFERED="1")
        self.proc = subprocess.Popen(
            [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(folder), "--dtype", dtype,
             "--out", str(self.out), "--max-tokens", str(max_tokens), "--page-size", str(page_size), *extra],
            stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True, env=env,
        )

    def step(self, entries, end=(), vocab=None):
        rec = {"step": self.step_no, "entries": entries, "end": list(end)}
        self.proc.stdin.write(json.dumps(rec) + "\n")
        self.proc.stdin.flush()
        line = self.proc.stdout.readline().strip()
        if line != f"done {self.step_no}":
            raise RuntimeError(f"trace_run answered {line!r} to step {self.step_no} (exit {self.proc.poll()})")
        path = self.out / f"{self.step_no}.f32"
        self.step_no += 1
        wanted = sum(len(e.get("want", [])) for e in entries)
        if not wanted:
            assert not path.exists()
            return None
        arr = np.fromfile(path, dtype="<f4")
        return torch.from_numpy(arr.reshape(wanted, -1).copy())

    def close(self) -> int:
        self.proc.stdin.close()
        code = self.proc.wait(timeout=120)
        return code

    def stats(self) -> dict:
        """What the program wrote when its input ended."""
        return json.loads((self.out / "stats.json").read_text())
