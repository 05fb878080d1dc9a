"""Command line in the reference's manner: ``demo``, ``generate`` and ``bench`` print one JSON report.

The reference's entry is ``mini-hisparse {demo,generate,bench}`` (mini_hisparse/cli.py:24-79).
Options it has keep their names and meanings here: --device, --gpu-pages, --page-size, --dtype,
--output, --max-new-tokens, --top-k (only ``all``: this engine attends to every key), --model,
--prompt, --chat, --requests, --prompt-tokens, --steps.  Options of its host-resident cache
(--host-pages, --eviction-policy, --hot-rows, ...) have no meaning here and are not offered.
Added: --temperature, --seed, --max-tokens-per-step, --prompt-ids / --prompt-file (token ids, so
that no tokenizer is needed), and for random weights --config and --weight-seed.
"""
from __future__ import annotations

import argparse
import json
import sys
import time
from pathlib import Path

DEMO_CONFIG = Path(__file__).resolve().parent / "configs" / "demo.json"


def _top_k(value):
    if value != "all":
        raise argparse.ArgumentTypeError("this engine attends to all keys: --top-k takes only 'all'")
    return None


def build_parser() -> argparse.ArgumentParser:
    parser = argparse.ArgumentParser(prog="mini_hisparse_b200",
                                     description="Qwen2 generation on one B200 with hand-written kernels")
    sub = parser.add_subparsers(dest="command", required=True)
    for name in ("demo", "generate", "bench"):
        c = sub.add_parser(name)
        c.add_argument("--device", default="cuda:0")
        c.add_argument("--gpu-pages", type=int, help="pages of the KV pool (default: what the requests need)")
        c.add_argument("--page-size", type=int, default=16)
        c.add_argument("--dtype", choices=["float32", "bfloat16"], default="float32")
        c.add_argument("--output", type=Path)
        c.add_argument("--max-tokens-per-step", type=int, default=2048)
        if name != "bench":
            c.add_argument("--top-k", type=_top_k, default=None, help="all (default)")
            c.add_argument("--max-new-tokens", type=int, default=12)
            c.add_argument("--temperature", type=float, default=0.0)
            c.add_argument("--seed", type=int, default=42)
        if name == "generate":
            c.add_argument("--model", required=True, help="folder with config.json and model.safetensors")
            c.add_argument("--prompt", help="text; needs a tokenizer in the model folder")
            c.add_argument("--prompt-ids", help="comma-separated token ids; ';' separates requests")
            c.add_argument("--prompt-file", type=Path, help="JSON list of token-id lists")
            c.add_argument("--chat", action="store_true", help="apply the tokenizer's chat template")
        else:
            c.add_argument("--config", type=Path, default=DEMO_CONFIG, help="config.json for random weights")
            c.add_argument("--weight-seed", type=int, default=42)
            c.add_argument("--requests", type=int, default=3)
        if name == "demo":
            c.add_argument("--prompt-tokens", type=int, default=65)
        if name == "bench":
            c.add_argument("--prompt-tokens", type=int, default=1024)
            c.add_argument("--steps", type=int, default=20)
            c.add_argument("--layers", type=int, help="run fewer layers than the config has")
            c.add_argument("--prefill", action="store_true",
                           help="time one prompt of --prompt-tokens in portions of --max-tokens-per-step instead of decoding")
    return parser


def _tokenizer(folder):
    try:
        from transformers import AutoTokenizer
    except Exception as e:   # noqa: BLE001
        raise SystemExit(f"--prompt needs a tokenizer library ({e}); give --prompt-ids instead")
    try:
        return AutoTokenizer.from_pretrained(str(folder), local_files_only=True)
    except Exception as e:   # noqa: BLE001
        raise SystemExit(f"no tokenizer could be loaded from {folder} ({e}); give --prompt-ids instead")


def _prompts_of(args, vocab):
    import torch

    if args.command == "generate":
        if args.prompt_ids:
            return [[int(t) for t in part.split(",") if t.strip()] for part in args.prompt_ids.split(";")], None
        if args.prompt_file:
            return json.loads(args.prompt_file.read_text()), None
        tok = _tokenizer(args.model)
        text = args.prompt or "Explain how a KV cache works."
        if args.chat:
            ids = tok.apply_chat_template([{"role": "user", "content": text}], tokenize=True,
                                          add_generation_prompt=True, return_dict=False)
        else:
            ids = tok.encode(text)
        return [list(ids)], tok
    if args.requests < 1 or args.prompt_tokens < 1:
        raise SystemExit("requests and prompt-tokens must be positive")
    g = torch.Generator().manual_seed(args.seed)
    # mini_hisparse/cli.py:126-133: request i has prompt_tokens + 7 i random tokens
    return [torch.randint(0, vocab, (args.prompt_tokens + 7 * i,), generator=g).tolist()
            for i in range(args.requests)], None


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    import torch

    from .engine.engine import Engine, load_model

    if args.command == "bench":
        from .measure import decode_benchmark, prefill_benchmark

        if args.prefill:
            result = prefill_benchmark(json.loads(args.config.read_text()), prompt_tokens=args.prompt_tokens,
                                       max_tokens_per_step=args.max_tokens_per_step, dtype=args.dtype,
                                       device=args.device, page_size=args.page_size, weight_seed=args.weight_seed,
                                       layers=args.layers)
            text = json.dumps(result, indent=2)
            if args.output:
                args.output.write_text(text + "\n")
            print(text)
            return 0
        result = decode_benchmark(json.loads(args.config.read_text()), batch=args.requests,
                                  prompt_tokens=args.prompt_tokens, steps=args.steps, dtype=args.dtype,
                                  device=args.device, page_size=args.page_size, weight_seed=args.weight_seed,
                                  layers=args.layers)
    else:
        if args.command == "generate":
            model = load_model(args.model, device=args.device, dtype=args.dtype)
            label = str(args.model)
        else:
            model = load_model(json.loads(args.config.read_text()), device=args.device, dtype=args.dtype,
                               random_seed=args.weight_seed)
            label = "random weights (mechanics demo)"
        prompts, tokenizer = _prompts_of(args, model.spec.vocab_size)
        need = sum(-(-(len(p) + args.max_new_tokens) // args.page_size) for p in prompts)
        engine = Engine(model, num_pages=args.gpu_pages or need, page_size=args.page_size,
                        max_requests=max(1, min(len(prompts), 64)),
                        max_tokens_per_step=args.max_tokens_per_step,
                        eos_token_id=tokenizer.eos_token_id if tokenizer else None)
        for i, prompt in enumerate(prompts):
            engine.add_request(str(i), prompt, args.max_new_tokens, temperature=args.temperature,
                               seed=args.seed + i)
        start = time.perf_counter()
        timeline = []
        while not engine.scheduler.idle:
            engine.step()
            timeline.append({
                "active": len(engine.running), "waiting": len(engine.waiting),
                "generated": {name: len(r.generated) for name, r in engine.requests.items()},
            })
        torch.cuda.synchronize()
        seconds = time.perf_counter() - start
        outputs = {name: r.generated for name, r in engine.requests.items()}
        result = {
            "model": label,
            "selection": "full attention",
            "outputs": {name: tokenizer.decode(t, skip_special_tokens=True) if tokenizer else t
                        for name, t in outputs.items()},
            "requests": {name: {"prefill_count": r.prefill_count, "decode_count": r.decode_count,
                                "generated_tokens": len(r.generated)}
                         for name, r in engine.requests.items()},
            "timeline": timeline,
            "seconds": seconds,
            "tokens_per_second": sum(map(len, outputs.values())) / seconds,
            **engine.snapshot(),
        }
        engine.cache.assert_invariants()
    text = json.dumps(result, indent=2, ensure_ascii=False)
    print(text)
    if args.output:
        args.output.parent.mkdir(parents=True, exist_ok=True)
        args.output.write_text(text + "\n")
    return 0


if __name__ == "__main__":
    sys.exit(main())
