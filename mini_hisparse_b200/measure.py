"""Measurement of the decode step and of a prompt's prefill: timing, byte and flop counts.

The reference measures only its storage path (experiments/benchmark.py:1, docs/benchmarks.md:88:
"not LLM tokens/s"); generation speed is this engine's own metric.  A decode step is timed on
the device with CUDA events around K consecutive steps of the engine's step function (graph
replay plus the copy of that step's index arrays); the end-to-end number goes through
``Engine.step()`` with host token lists in and out.  Every step reads all weights (far more than
the L2 holds), so no L2 flush is needed between steps.
"""
from __future__ import annotations

import json
import subprocess
import time
from pathlib import Path

import torch

from .kernels import api as K

ROOT = Path(__file__).resolve().parent.parent
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0,
                  "source": "fallback"}


def peaks() -> dict:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            d = json.loads(path.read_text())
            out = {"source": "measured"}
            for k in ("hbm_gbs", "bf16_tflops", "bf16_tflops_sustained"):
                out[k] = float(d[k]) if k in d else FALLBACK_PEAKS[k]
            return out
        except Exception:   # noqa: BLE001
            pass
    return dict(FALLBACK_PEAKS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while a region runs."""

    QUERY = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int = 0):
        self.proc = None
        self.index = index

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", "100"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
        return self

    def __exit__(self, *exc):
        self.result = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return
        self.proc.terminate()
        try:
            out, _ = self.proc.communicate(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
            out, _ = self.proc.communicate()
        clocks, reasons, mx = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in out.splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 7:
                continue
            try:
                clocks.append(float(parts[0]))
                mx = float(parts[1])
            except ValueError:
                continue
            for n, v in zip(names, parts[3:7]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if clocks:
            clocks.sort()
            self.result = {"sm_mhz": clocks[len(clocks) // 2], "sm_max_mhz": mx,
                           "reasons": sorted(reasons), "samples": len(clocks)}


# ---- counts -------------------------------------------------------------------------------------
def decode_bytes(model, cache, live_tokens: int) -> int:
    """Bytes a decode step has to read: every weight it uses once (the embedding table is only
    gathered, so it does not count unless it is also the tied head) and the cache of the live
    requests."""
    weights = model.weight_bytes()
    emb = model.embedding.weight
    if model.head.weight.data_ptr() != emb.data_ptr():
        weights -= emb.numel() * emb.element_size()
    kv = 0
    for g in cache.page_groups:
        kv += g.page_bytes() // cache.cfg.page_size * live_tokens
    return weights + kv


def prefill_flops(cfg, layers: int, T: int) -> float:
    """2 flops per weight element per token for the products, 4 nq d per (query, key) pair for
    causal attention (half of T^2 pairs)."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_token = 2 * (H * (q + 2 * kv) + q * H + 3 * H * I)
    attn = 4 * cfg.num_attention_heads * cfg.head_dim * T * (T + 1) / 2
    return layers * (per_token * T + attn) + 2 * H * V     # the head runs on the last row only


# ---- building ---------------------------------------------------------------------------------
def build_engine(config: dict, *, batch: int, context: int, dtype="bfloat16", device="cuda:0",
                 page_size=16, weight_seed=0, layers: int | None = None, max_tokens_per_step=2048,
                 extra_pages: int = 0):
    from .engine.engine import Engine, load_model

    config = dict(config)
    if layers is not None:
        config["num_hidden_layers"] = layers
    model = load_model(config, device=device, dtype=dtype, random_seed=weight_seed)
    pages = batch * -(-context // page_size) + extra_pages
    engine = Engine(model, num_pages=pages, page_size=page_size, max_requests=batch,
                    max_tokens_per_step=max_tokens_per_step)
    return engine


def synthetic_context(engine, batch: int, tokens: int, seed: int = 0) -> list[str]:
    """Open ``batch`` requests that already hold ``tokens`` cached positions each.  The pages are
    filled with random keys and values instead of running prompts through the model: like the
    weights, the cache content is synthetic, and a decode step's cost does not depend on it."""
    cache = engine.cache
    names = []
    gen = torch.Generator(device=cache.cfg.device).manual_seed(seed)
    for g in cache.page_groups:
        g.storage.normal_(0.0, 0.5, generator=gen)
    for i in range(batch):
        name = f"bench{i}"
        cache.open(name)
        cache.ensure(name, tokens)
        cache.advance(name, tokens)
        names.append(name)
    return names


def time_decode(engine, names, steps: int, warmup: int, vocab: int, sampled_warmup: int = 0) -> dict:
    """Device time of ``steps`` decode steps of the step function (one token per request).

    The clocks are sampled every 100 ms (more often disturbs the timing), so a short timed region may
    see no sample: ``sampled_warmup`` further untimed steps of the same load run between the warm-up
    and the timed steps with the sampler already on."""
    from .engine.step import StepEntry

    B = len(names)
    gen = torch.Generator().manual_seed(1)
    def entries():
        toks = torch.randint(0, vocab, (B,), generator=gen).tolist()
        return [StepEntry(n, [t], [0]) for n, t in zip(names, toks)]
    for _ in range(warmup):
        engine.runner.step(entries())
    torch.cuda.synchronize()
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = K.launches
    with ClockSampler() as clocks:
        for _ in range(sampled_warmup):
            engine.runner.step(entries())
        launches0 = K.launches
        torch.cuda.synchronize()
        start.record()
        for _ in range(steps):
            engine.runner.step(entries())
        end.record()
        torch.cuda.synchronize()
    ms = start.elapsed_time(end)
    engine.runner.check_status()
    return {"ms_per_step": ms / steps, "tokens_per_s": B * steps / (ms / 1e3),
            "launches": K.launches - launches0, "clocks": clocks.result}


def decode_benchmark(config: dict, *, batch=8, prompt_tokens=1024, steps=20, warmup=3,
                     dtype="bfloat16", device="cuda:0", page_size=16, weight_seed=0,
                     layers: int | None = None) -> dict:
    """What ``bench`` of the command line prints: decode tokens a second at one batch size."""
    engine = build_engine(config, batch=batch, context=prompt_tokens + steps + warmup + 1, dtype=dtype,
                          device=device, page_size=page_size, weight_seed=weight_seed, layers=layers)
    names = synthetic_context(engine, batch, prompt_tokens)
    r = time_decode(engine, names, steps, warmup, engine.model.spec.vocab_size)
    live = batch * (prompt_tokens + warmup + steps // 2)
    nbytes = decode_bytes(engine.model, engine.cache, live)
    p = peaks()
    gbs = nbytes / (r["ms_per_step"] / 1e3) / 1e9
    return {"metric": "decode tokens/s", "batch": batch, "context": prompt_tokens, "dtype": dtype,
            "tokens_per_second": r["tokens_per_s"], "ms_per_step": r["ms_per_step"],
            "bytes_per_step": nbytes, "achieved_gbs": gbs,
            "hbm_fraction": gbs / p["hbm_gbs"], "peak_source": p["source"], "clocks": r["clocks"]}
