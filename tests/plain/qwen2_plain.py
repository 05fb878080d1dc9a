"""Plain, slow Qwen2 forward pass: whole sequences, no cache, one function per part.

This file is the oracle of the test-suite.  It is written from the formulas of
KiritoHugh/mini-hisparse (cited per function as ``file:line`` within that
project) and shares no code with the engine package: it has its own reader for
the model folder, its own configuration parsing and its own sampling draw.
``tests/golden/`` holds outputs of the reference's own model code on a tiny
random model, and ``tests/test_plain.py`` compares this file with them, so the
oracle rests on the reference's code and not only on its formulas.

Everything runs in the dtype it is given (float32 or float64 on the CPU; the
GPU tests also run it in float32 on the device at large sizes).

``act``: the functions that end a part take an optional dtype to which that part's
output is rounded (and widened again), so that a float32 run can stand in for a
model whose activations between the parts are bfloat16 while every sum stays
float32: normalised rows, rotated q and k, v, the attention output and the gated
feed-forward activation.  The reference rounds at the same places when its model
dtype is bfloat16 (model.py:51, 138-153, 179, 71); with ``act=None`` nothing is rounded.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import torch

_ST_DTYPES = {
    "F64": torch.float64,
    "F32": torch.float32,
    "F16": torch.float16,
    "BF16": torch.bfloat16,
    "I64": torch.int64,
    "I32": torch.int32,
}


def read_safetensors(path) -> dict[str, torch.Tensor]:
    """Minimal reader: 8-byte little-endian header length, JSON header, raw data."""
    blob = Path(path).read_bytes()
    (n,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + n])
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        begin, end = meta["data_offsets"]
        raw = bytearray(blob[8 + n + begin : 8 + n + end])
        dtype = _ST_DTYPES[meta["dtype"]]
        if len(raw) == 0:
            out[name] = torch.empty(meta["shape"], dtype=dtype)
        else:
            out[name] = torch.frombuffer(raw, dtype=dtype).reshape(meta["shape"]).clone()
    return out


class PlainConfig:
    """The keys of config.json that the formulas need (model.py:19-40, 103-123)."""

    def __init__(self, d: dict):
        self.vocab_size = d["vocab_size"]
        self.hidden_size = d["hidden_size"]
        self.intermediate_size = d["intermediate_size"]
        self.num_hidden_layers = d["num_hidden_layers"]
        self.num_attention_heads = d["num_attention_heads"]
        self.num_key_value_heads = d.get("num_key_value_heads", self.num_attention_heads)
        # model.py:30-32: head_dim = hidden_size // num_attention_heads; an explicit key wins.
        self.head_dim = d.get("head_dim") or self.hidden_size // self.num_attention_heads
        self.rms_norm_eps = d["rms_norm_eps"]
        rope = d.get("rope_parameters") or d.get("rope_scaling") or {}
        self.rope_theta = rope.get("rope_theta", d.get("rope_theta"))
        self.tie_word_embeddings = bool(d.get("tie_word_embeddings", False))


def load_folder(folder, dtype=torch.float32, device="cpu"):
    folder = Path(folder)
    cfg = PlainConfig(json.loads((folder / "config.json").read_text()))
    weights = {
        k: v.to(dtype=dtype, device=device)
        for k, v in read_safetensors(folder / "model.safetensors").items()
    }
    if cfg.tie_word_embeddings and "lm_head.weight" not in weights:
        weights["lm_head.weight"] = weights["model.embed_tokens.weight"]
    return cfg, weights


# ---------------------------------------------------------------------------
# parts
# ---------------------------------------------------------------------------

def _rounded(t: torch.Tensor, act) -> torch.Tensor:
    return t if act is None else t.to(act).to(t.dtype)


def embedding(tokens: torch.Tensor, table: torch.Tensor) -> torch.Tensor:
    """model.py:166 — plain row lookup, no scaling."""
    return table[tokens]


def rms_norm(x: torch.Tensor, weight: torch.Tensor, eps: float, act=None) -> torch.Tensor:
    """model.py:49-51 — x * rsqrt(mean(x^2) + eps), then times the weight."""
    xf = x.float() if x.dtype in (torch.float16, torch.bfloat16) else x
    n = xf * torch.rsqrt(xf.square().mean(-1, keepdim=True) + eps)
    return _rounded(n.to(x.dtype) * weight, act)


def linear(x, weight, bias=None):
    """nn.Linear of model.py:57-60, 66-68, 96: y = x W^T + b."""
    y = x @ weight.transpose(0, 1)
    return y if bias is None else y + bias


def rope_tables(positions: torch.Tensor, head_dim: int, theta: float, dtype):
    """model.py:141-147 — inv = theta^(-(2i)/d) in float32, angles = p * inv, both halves alike."""
    inv = theta ** (-torch.arange(0, head_dim, 2, device=positions.device).float() / head_dim)
    angles = positions.float()[:, None] * inv[None, :]
    angles = torch.cat((angles, angles), -1)[:, None, :]
    return angles.cos().to(dtype), angles.sin().to(dtype)


def rotate(t: torch.Tensor, cosine, sine) -> torch.Tensor:
    """model.py:149-151 — half-split rotation: t*cos + cat(-t[d/2:], t[:d/2])*sin."""
    a, b = t.chunk(2, -1)
    return t * cosine + torch.cat((-b, a), -1) * sine


def causal_attention(q, k, v, window: int | None = None) -> torch.Tensor:
    """model.py:173-179 (SDPA, is_causal) spelled out as selection.py:158-163 does:
    query head h reads KV head h // groups, scores / sqrt(d), softmax over keys <= own position.

    q [T, nq, d]; k, v [T, nkv, d] -> [T, nq, d].  ``window`` (not a Qwen2 option) keeps the
    last ``window`` keys only; it exists to test the kernels' window argument.
    """
    T, nq, d = q.shape
    groups = nq // k.shape[1]
    k = k.repeat_interleave(groups, 1)
    v = v.repeat_interleave(groups, 1)
    scores = torch.einsum("qhd,khd->hqk", q.float(), k.float()) / math.sqrt(d)
    qpos = torch.arange(T, device=q.device)[:, None]
    kpos = torch.arange(T, device=q.device)[None, :]
    mask = kpos > qpos
    if window is not None:
        mask = mask | (kpos <= qpos - window)
    scores = scores.masked_fill(mask[None], -torch.inf)
    out = torch.einsum("hqk,khd->qhd", scores.softmax(-1), v.float())
    return out.to(q.dtype)


def swiglu(x, gate_w, up_w, down_w, act=None):
    """model.py:70-71 — down(silu(gate(x)) * up(x))."""
    g = linear(x, gate_w)
    return linear(_rounded(g * torch.sigmoid(g) * linear(x, up_w), act), down_w)


def attention_block(cfg, w, prefix, x, positions, act=None):
    """model.py:135-153 (project + rotate) and 173-179 (attend) and o_proj of 157."""
    T = x.shape[0]
    q = linear(x, w[prefix + "q_proj.weight"], w[prefix + "q_proj.bias"])
    k = linear(x, w[prefix + "k_proj.weight"], w[prefix + "k_proj.bias"])
    v = linear(x, w[prefix + "v_proj.weight"], w[prefix + "v_proj.bias"])
    q = q.view(T, cfg.num_attention_heads, cfg.head_dim)
    k = k.view(T, cfg.num_key_value_heads, cfg.head_dim)
    v = v.view(T, cfg.num_key_value_heads, cfg.head_dim)
    cosine, sine = rope_tables(positions, cfg.head_dim, cfg.rope_theta, x.dtype)
    q, k, v = _rounded(rotate(q, cosine, sine), act), _rounded(rotate(k, cosine, sine), act), _rounded(v, act)
    a = _rounded(causal_attention(q, k, v), act)
    return linear(a.reshape(T, -1), w[prefix + "o_proj.weight"])


def decoder_layer(cfg, w, index, x, positions, act=None):
    """model.py:155-158 — pre-norm residual block."""
    p = f"model.layers.{index}."
    h = rms_norm(x, w[p + "input_layernorm.weight"], cfg.rms_norm_eps, act)
    x = x + attention_block(cfg, w, p + "self_attn.", h, positions, act)
    h = rms_norm(x, w[p + "post_attention_layernorm.weight"], cfg.rms_norm_eps, act)
    return x + swiglu(
        h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"], act
    )


@torch.inference_mode()
def forward_logits(cfg, w, tokens, act=None) -> torch.Tensor:
    """Logits at EVERY position of one whole sequence, float32 [T, V]
    (model.py:160-181 returns the last row only; the rows are independent of that choice)."""
    table = w["model.embed_tokens.weight"]
    tokens = torch.as_tensor(tokens, dtype=torch.long, device=table.device)
    positions = torch.arange(len(tokens), device=table.device)
    x = embedding(tokens, table)
    for i in range(cfg.num_hidden_layers):
        x = decoder_layer(cfg, w, i, x, positions, act)
    x = rms_norm(x, w["model.norm.weight"], cfg.rms_norm_eps, act)
    return linear(x, w["lm_head.weight"]).float()


# ---------------------------------------------------------------------------
# sampling
# ---------------------------------------------------------------------------

def greedy(logits: torch.Tensor) -> int:
    """engine.py:72 — argmax, lowest index on ties."""
    return int(logits.argmax().item())


def uniform_from_counter(seed: int, counter: int) -> float:
    """The draw's uniform number in [0, 1): a 64-bit mix of (seed, counter), top 24 bits.

    The reference samples greedily only (engine.py:72); temperature sampling is this
    engine's own, so this is its definition: splitmix64 of seed * 0x9E3779B97F4A7C15 + counter.
    """
    mask = (1 << 64) - 1
    z = (seed * 0x9E3779B97F4A7C15 + counter + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return (z >> 40) / float(1 << 24)


def sample_temperature(logits: torch.Tensor, temperature: float, seed: int, counter: int):
    """softmax(logits / temperature) in float64, inverse CDF at the counter's uniform number.

    Returns (token, margin): margin is the distance of the uniform number to the nearest
    CDF edge of the chosen token, so a test can tell a rounding tie from a fault.
    """
    p = (logits.double() / temperature).softmax(-1)
    cdf = p.cumsum(-1)
    u = uniform_from_counter(seed, counter) * float(cdf[-1])
    token = int(torch.searchsorted(cdf, torch.tensor(u, dtype=torch.float64), right=True).item())
    token = min(token, logits.numel() - 1)
    low = float(cdf[token - 1]) if token else 0.0
    return token, min(u - low, float(cdf[token]) - u)


@torch.inference_mode()
def generate(cfg, w, prompt, max_new_tokens, temperature=0.0, seed=0, eos_token_id=None):
    """engine.py:71-77 restated: re-run the whole history for every token."""
    history, out = list(prompt), []
    for i in range(max_new_tokens):
        logits = forward_logits(cfg, w, history)[-1]
        token = greedy(logits) if temperature == 0 else sample_temperature(logits, temperature, seed, i)[0]
        out.append(token)
        history.append(token)
        if token == eos_token_id:
            break
    return out
