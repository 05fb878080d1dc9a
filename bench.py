#!/usr/bin/env python3
"""Decode throughput of the engine at Qwen2.5-7B shape with random weights, on one GPU.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--impl ours|reference]

Prints ONE JSON line.  ``value`` is decoded tokens a second at batch 8 with about 4,096 tokens of
context per request, timed on the device around K decode steps of the step function;
``e2e`` is the same through ``Engine.step()`` with host token ids in and sampled host tokens
out (its prompts are really prefilled); ``prefill`` times a 2,048-token prompt; ``roofline``
relates the decode step to the bytes it has to read; ``points`` holds batch 1 and 64.
For --gpus > 1 it prints one line that says so and exits with 2: this engine is single-GPU.

    python bench.py --workload serving14b|long32b [--layers L]

runs one of the two serving workloads instead and prints ITS one JSON line: 32 requests with prompts
of 128 to 4,096 tokens in portions of 512 beside decoding at the Qwen2.5-14B shape, or 16 requests of
8,192 prompt tokens plus 512 generated ones at the Qwen2.5-32B shape with the page pool sized from
free memory; tokens a second, step-time percentiles, roofline fractions, clocks, and the layer count.
"""
from __future__ import annotations

import argparse
import gc
import json
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

# BASELINE.json configs[2]: Qwen2.5-7B shape, kept as data beside the package
CONFIG_7B = json.loads((ROOT / "mini_hisparse_b200" / "configs" / "qwen2.5-7b-shape.json").read_text())
WORKLOADS = {"serving14b": "qwen2.5-14b-shape.json", "long32b": "qwen2.5-32b-shape.json"}
CONTEXT = 4096
PREFILL_TOKENS = 2048
PAGE = 16
SAMPLED = 64       # untimed decode steps under the clock sampler before the timed ones


def reference_arm(args) -> int:
    from baseline.reference_arm import run_reference

    print(json.dumps(run_reference(CONFIG_7B, CONTEXT, args)))
    return 0


def workload(args) -> int:
    from mini_hisparse_b200 import measure

    config = json.loads((ROOT / "mini_hisparse_b200" / "configs" / WORKLOADS[args.workload]).read_text())
    prompts, settings = measure.workload_prompts(args.workload, config["vocab_size"])
    line = measure.serving_workload(config, prompts=prompts, layers=args.layers, page_size=PAGE,
                                    label=args.workload, graph_after=args.graph_after, **settings)
    line = {"metric": f"tokens/s of the {args.workload} workload (prompt and generated, through Engine.step)",
            "value": line["tokens_per_s"], "unit": "tokens/s", "n_gpus": 1, "higher_is_better": True, "impl": "ours",
            **line}
    print(json.dumps(line))
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None,
                    help="timed decode steps (default 64; 4 for the reference arm, whose steps take seconds)")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=None, help="run fewer layers than the 28 of the config")
    ap.add_argument("--no-points", action="store_true", help="skip batch 1 and 64")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), help="run a serving workload instead of the decode bench")
    ap.add_argument("--graph-after", type=int, default=8,
                    help="with --workload: capture a decode graph at the N-th step that asks for it")
    args = ap.parse_args()
    if args.gpus != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    if args.steps is None:
        args.steps = 4 if args.impl == "reference" else 64
    if args.impl == "reference":
        return reference_arm(args)
    args.warmup = max(args.warmup, 3)
    if args.workload:
        return workload(args)

    import torch

    from mini_hisparse_b200 import measure
    from mini_hisparse_b200.config import Qwen2Config
    from mini_hisparse_b200.engine.engine import Engine, load_model
    from mini_hisparse_b200.engine.step import StepEntry
    from mini_hisparse_b200.kernels import api as K

    cfg_dict = dict(CONFIG_7B)
    layers = args.layers or cfg_dict["num_hidden_layers"]
    cfg_dict["num_hidden_layers"] = layers
    cfg = Qwen2Config.from_dict(cfg_dict)
    model = load_model(cfg_dict, device="cuda:0", dtype="bfloat16", random_seed=0)
    peaks = measure.peaks()
    vocab = cfg.vocab_size
    steps, warmup = args.steps, args.warmup
    # What follows a prefill (the end-to-end run's prompts, the 2,048-token prefill) starts under the
    # power cap that the prefill left behind: its first two dozen decode steps run at lower clocks.
    # Those measurements get more untimed steps, so that the timed ones are in the steady state.
    settle = max(warmup, 32)

    def decode_point(batch: int, warm: int = warmup) -> dict:
        # SAMPLED more untimed steps run before the timed ones with the clock sampler on, so that a
        # short timed region still has clock samples of its load
        start_ctx = CONTEXT - steps - warm - SAMPLED - 1      # the timed steps end at the context length
        engine = Engine(model, num_pages=batch * (CONTEXT // PAGE + 1), page_size=PAGE, max_requests=batch)
        names = measure.synthetic_context(engine, batch, start_ctx)
        r = measure.time_decode(engine, names, steps, warm, vocab, sampled_warmup=SAMPLED)
        live = batch * (start_ctx + warm + SAMPLED + steps // 2)
        r["bytes"] = measure.decode_bytes(model, engine.cache, live)
        del engine
        gc.collect()
        torch.cuda.empty_cache()
        return r

    main_pt = decode_point(args.batch)
    gbs = main_pt["bytes"] / (main_pt["ms_per_step"] / 1e3) / 1e9

    # ---- end to end through Engine.step(): host tokens in, host tokens out -------------------
    e2e = None
    if not args.no_e2e:
        engine = Engine(model, num_pages=args.batch * (CONTEXT // PAGE + 1), page_size=PAGE,
                        max_requests=args.batch, max_tokens_per_step=4096)
        g = torch.Generator().manual_seed(3)
        # prompts finish their prefill one step after the other: the first request decodes up to
        # `batch` tokens before the last one starts, so everyone gets that many tokens more
        budget = steps + settle + args.batch + 2
        for i in range(args.batch):
            prompt = torch.randint(0, vocab, (CONTEXT - budget,), generator=g).tolist()
            engine.add_request(f"e{i}", prompt, max_new_tokens=budget)
        while not all(r.decoding for r in engine.requests.values()):
            engine.step()                           # real prefill, untimed
        torch.cuda.synchronize()
        done = 0
        stamps = []
        for i in range(settle + steps):
            if i == settle:
                torch.cuda.synchronize()
                t0 = time.perf_counter()
            n = len(engine.step())
            stamps.append(time.perf_counter())
            if i >= settle:
                done += n
        torch.cuda.synchronize()
        sec = time.perf_counter() - t0
        print("e2e step times (ms):", [round((b - a) * 1e3, 2) for a, b in zip(stamps, stamps[1:])],
              file=sys.stderr)
        # per step: the packed index arrays go up from pinned memory, the sampled ids come down
        words = engine.runner.graphs[next(iter(engine.runner.graphs))].layout.total if engine.runner.graphs else 0
        e2e = {"value": done / sec, "unit": "tokens/s", "h2d_bytes_per_step": words * 4,
               "d2h_bytes_per_step": 4 * args.batch + 4, "ms_per_step": sec / steps * 1e3, "warmup": settle}
        del engine
        gc.collect()
        torch.cuda.empty_cache()

    # ---- prefill of one 2,048-token prompt -----------------------------------------------------
    engine = Engine(model, num_pages=PREFILL_TOKENS // PAGE + 8, page_size=PAGE, max_requests=2,
                    max_tokens_per_step=PREFILL_TOKENS)
    g = torch.Generator().manual_seed(5)
    times = []
    for i in range(4):
        name = f"p{i}"
        engine.cache.open(name)
        toks = torch.randint(0, vocab, (PREFILL_TOKENS,), generator=g).tolist()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        engine.runner.step([StepEntry(name, toks, [PREFILL_TOKENS - 1])])
        b.record()
        torch.cuda.synchronize()
        times.append(a.elapsed_time(b))
        engine.cache.close(name)
    pre_ms = min(times[1:])
    flops = measure.prefill_flops(cfg, layers, PREFILL_TOKENS)
    prefill = {"value": PREFILL_TOKENS / (pre_ms / 1e3), "tokens": PREFILL_TOKENS, "ms": pre_ms,
               "frac": flops / (pre_ms / 1e3) / (peaks["bf16_tflops"] * 1e12), "tflops": flops / (pre_ms / 1e3) / 1e12}
    del engine
    gc.collect()
    torch.cuda.empty_cache()

    points = {}
    if not args.no_points:
        for b in (1, 64):
            points[f"decode_b{b}"] = decode_point(b, settle)["tokens_per_s"]

    line = {
        "metric": "decode tokens/s (Qwen2.5-7B shape, batch 8, context 4096)",
        "value": main_pt["tokens_per_s"],
        "unit": "tokens/s",
        "n_gpus": 1,
        "steps": steps,
        "warmup": warmup,
        "ms_per_step": main_pt["ms_per_step"],
        "higher_is_better": True,
        "scaling": "weak",
        "vs_baseline": None,
        "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform-random token ids, random KV for the device-timed context",
        "impl": "ours",
        "config": measure.headline_config(CONFIG_7B, batch=args.batch, context=CONTEXT, layers=layers, page_size=PAGE),
        "clocks": main_pt["clocks"],
        "e2e": e2e,
        "gpu_launches": main_pt["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                     "frac": gbs / peaks["hbm_gbs"]},
        "points": points,
    }
    print(json.dumps(line))
    return 0


if __name__ == "__main__":
    sys.exit(main())
