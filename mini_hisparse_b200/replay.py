"""Replay given token ids through a model step by step and write the logits that are asked for.

    bin/trace_run --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N

Steps come from standard input, one JSON object a line:

    {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": []}

All entries of a step run as ONE batch through the engine's own step function (the model,
cache manager and kernels that generation uses); nothing is sampled.  For a step that wants
logits, ``OUT/<step>.f32`` receives them as little-endian float32 [wanted, vocab], in the order
of the entries and of their ``want`` lists.  After every step the program prints ``done <step>``
and flushes.  Requests named in ``end`` give back what they hold after the step.  The cache pool
is sized for --max-tokens (each request's tokens rounded up to a multiple of 64, or of the page
size if that is larger), so pages are used again.  Exit status 0 when the input ends.

A step of single tokens that all want their logits goes the way the engine's decode steps go:
through a CUDA graph captured for its batch size (--no-graphs launches it eagerly instead), with
its index arrays packed ahead of time when the step before it had the same requests.  When the
input ends, the runner's counters (steps, graph_steps, prepared_steps, ...) and the cache's are
written to ``OUT/stats.json``.  --poison overwrites every page that is given back, so that a
read of a stale page cannot pass for a right one.

The reference's replay (experiments/replay.py:19-151) feeds frozen per-layer Q/K/V through a
cache and checks attention outputs; this one replays tokens through the whole model.
"""
import argparse
import json
import sys
from pathlib import Path


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    ap.add_argument("--out", required=True, help="folder for <step>.f32 files")
    ap.add_argument("--max-tokens", type=int, required=True,
                    help="most tokens that live requests hold at any time (rounded up per request)")
    ap.add_argument("--page-size", type=int, default=16)
    ap.add_argument("--max-requests", type=int, default=8)
    ap.add_argument("--device", default="cuda:0")
    ap.add_argument("--no-graphs", dest="graphs", action="store_false",
                    help="launch decode steps eagerly instead of replaying a captured CUDA graph")
    ap.add_argument("--poison", action="store_true", help="overwrite pages that are given back")
    args = ap.parse_args()

    print("[trace_run] loading (the first call compiles the CUDA kernels this model needs)",
          file=sys.stderr, flush=True)
    import numpy as np
    import torch

    from .cache.manager import CacheConfig, CacheManager
    from .engine.engine import load_model, parse_dtype
    from .engine.step import ModelRunner, StepEntry

    if not torch.cuda.is_available():
        print("trace_run: no CUDA device is visible; this engine has no CPU path", file=sys.stderr)
        return 3
    out = Path(args.out)
    out.mkdir(parents=True, exist_ok=True)
    dtype = parse_dtype(args.dtype)
    model = load_model(args.model, device=args.device, dtype=dtype)
    page = args.page_size
    if page < 1:
        print("trace_run: --page-size must be positive", file=sys.stderr)
        return 2
    # --max-tokens counts every live request's tokens rounded up to a multiple of 64 (of the page
    # size, if that is larger): a unit of 64 tokens takes ceil(64 / page) pages whatever the page size
    if page >= 64:
        num_pages = -(-args.max_tokens // page)
    else:
        num_pages = -(-args.max_tokens // 64) * -(-64 // page)
    cache = CacheManager(
        model.cache_needs,
        CacheConfig(num_pages=max(1, num_pages), page_size=page, max_requests=args.max_requests,
                    dtype=dtype, device=args.device, debug_poison=args.poison),
    )
    try:
        runner = ModelRunner(model, cache, use_graphs=args.graphs)
    except ValueError as e:        # a part that cannot work over this cache says so before any step
        print(f"trace_run: {e}", file=sys.stderr)
        return 2
    print("[trace_run] ready", file=sys.stderr, flush=True)

    for line in sys.stdin:
        line = line.strip()
        if not line:
            continue
        rec = json.loads(line)
        step = rec["step"]
        entries = []
        for e in rec.get("entries", []):
            rid = e["id"]
            if rid not in cache.requests:
                cache.open(rid)
            entries.append(StepEntry(rid, list(e["tokens"]), list(e.get("want", []))))
        logits = runner.step(entries) if entries else None
        ended = set(rec.get("end", []))
        if entries and all(len(e.tokens) == 1 and e.want == [0] for e in entries) and not ended:
            # while the GPU runs this step: pack the next one's index arrays, guessing that it decodes
            # the same requests (dropped if it does not); no page is taken early, the pool is tight
            runner.prepare_decode_ahead([e.request for e in entries], take_pages=False)
        if logits is not None:
            arr = logits.detach().to("cpu", torch.float32).contiguous().numpy()
            arr.astype("<f4", copy=False).tofile(out / f"{step}.f32")
        runner.check_status()
        for rid in rec.get("end", []):
            if rid in cache.requests:
                cache.close(rid)
        print(f"done {step}", flush=True)
    cache.assert_invariants()
    (out / "stats.json").write_text(json.dumps({"runner": runner.stats, "cache": cache.snapshot()}) + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
