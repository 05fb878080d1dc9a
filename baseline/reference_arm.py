"""The reference arm of bench.py: the UNMODIFIED KiritoHugh/mini-hisparse, installed into
``baseline/_ref`` with pip (--no-index --no-deps --target), driven through its own public API:
``MiniModel(ModelConfig(...))``, ``reference.cache.PagedKVCache(PagedConfig(...))``,
``Engine.add_request`` and ``Engine.step`` (mini_hisparse/engine.py:24-135), the way its command
line builds them for ``--cache-layout pages`` (mini_hisparse/cli.py:126-175) with every page
resident on the GPU.  None of this repository's model, kernels or engine is on that path.

The reference decodes one token of one request at a time (engine.py:80-84); a "step" is one
``Engine.step()``, which gives each of the B running requests one decode turn.
"""
from __future__ import annotations

import sys
import time
from pathlib import Path

REF = Path(__file__).resolve().parent / "_ref"


def run_reference(config: dict, context: int, args) -> dict:
    if not (REF / "mini_hisparse").is_dir():
        return {"impl": "reference", "unavailable": "baseline/_ref is not installed (pip install --no-index "
                "--no-deps --target baseline/_ref of the reference was not run on this checkout)"}
    try:
        return _run(config, context, args)
    except Exception as e:   # noqa: BLE001
        return {"impl": "reference", "unavailable": f"{type(e).__name__}: {str(e)[:300]}"}


def _run(config: dict, context: int, args) -> dict:
    sys.path.insert(0, str(REF))
    import torch
    from mini_hisparse.engine import Engine
    from mini_hisparse.model import MiniModel, ModelConfig
    from reference.cache import PagedConfig, PagedKVCache

    from mini_hisparse_b200.measure import ClockSampler, headline_config

    steps, warmup, batch = args.steps, max(args.warmup, 3), args.batch
    layers = args.layers or config["num_hidden_layers"]
    page = 16
    torch.manual_seed(42)
    cfg = ModelConfig(
        vocab_size=config["vocab_size"], hidden_size=config["hidden_size"],
        intermediate_size=config["intermediate_size"], num_hidden_layers=layers,
        num_attention_heads=config["num_attention_heads"],
        num_key_value_heads=config["num_key_value_heads"], rms_norm_eps=config["rms_norm_eps"],
        rope_theta=config["rope_theta"],
    )
    with torch.device("cuda:0"):
        model = MiniModel(cfg)
    model = model.eval().to(device="cuda:0", dtype=torch.bfloat16)
    start_ctx = context - steps - warmup - batch - 2
    pages = batch * layers * (context // page + 1)
    cache = PagedKVCache(PagedConfig(
        gpu_pages=pages, host_pages=pages, page_size=page, kv_heads=cfg.num_key_value_heads,
        head_dim=cfg.head_dim, device="cuda:0", dtype=torch.bfloat16,
        index_budget_bytes=8 * 1024 ** 3,
        # one attention window over the whole history (its --chunk-pages option): with the default
        # of 4 pages a decode step of this size took 27 s on a B200
        chunk_pages=context // page + 1,
    ))
    engine = Engine(model, cache)
    g = torch.Generator().manual_seed(3)
    for i in range(batch):
        prompt = torch.randint(0, cfg.vocab_size, (start_ctx,), generator=g).tolist()
        engine.add_request(str(i), prompt, steps + warmup + batch + 2)
    while engine.waiting:                 # one prompt is admitted and prefilled per step
        engine.step()
    for _ in range(warmup):
        engine.step()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    done = 0
    with ClockSampler() as clocks:
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        a.record()
        for _ in range(steps):
            done += len(engine.step())
        b.record()
        torch.cuda.synchronize()
        wall = time.perf_counter() - t0
    ms = a.elapsed_time(b)
    return {
        "impl": "reference",
        "metric": "decode tokens/s (Qwen2.5-7B shape, batch 8, context 4096)",
        "value": done / (ms / 1e3), "unit": "tokens/s", "n_gpus": 1, "steps": steps, "warmup": warmup,
        "ms_per_step": ms / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: torch default init, uniform-random token ids; reference.cache.PagedKVCache, all pages resident",
        "config": headline_config(config, batch=batch, context=context, layers=layers, page_size=page),
        "clocks": clocks.result,
        "e2e": {"value": done / wall, "unit": "tokens/s", "h2d_bytes_per_step": 8 * batch,
                "d2h_bytes_per_step": 8 * batch},
        "gpu_launches": None,
    }
