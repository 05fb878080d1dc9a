"""Generation through the Python entry point and the command line, against the plain
implementation: greedy, temperature, long decoding, the first tokens of a sequence, and what
happens when pages run out."""
import json
import subprocess
import sys

import pytest
import torch

from conftest import ROOT, TINY, random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu


def load(folder, dtype):
    from mini_hisparse_b200 import load_model

    return load_model(folder, device="cuda:0", dtype=dtype)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B"])
def test_greedy_generation_equals_plain(folders, name, dtype):
    from mini_hisparse_b200 import Engine

    cfg, page = TINY[name]
    pc, w = P.load_folder(folders[name])
    model = load(folders[name], dtype)
    # graph_after=2: a batch's first decode step runs launch by launch, the later ones from its graph
    engine = Engine(model, num_pages=64, page_size=page, max_requests=4, max_tokens_per_step=48, graph_after=2)
    prompts = {str(n): random_tokens(cfg["vocab_size"], n, seed=n) for n in (7, 33, 64)}
    for rid, prompt in prompts.items():
        engine.add_request(rid, prompt, max_new_tokens=16)
    out = engine.run()
    for rid, prompt in prompts.items():
        want = P.generate(pc, w, prompt, 16)
        if dtype == "float32":
            assert out[rid] == want
        else:
            # bfloat16 may flip a near-tie; up to there the tokens are equal, and the flip is a near-tie
            same = next((i for i, (a, b) in enumerate(zip(out[rid], want)) if a != b), 16)
            if same < 16:
                logits = P.forward_logits(pc, w, prompt + want[:same])[-1]
                top = logits.topk(2).values
                assert float(top[0] - top[1]) < 0.05 * float(logits.abs().max()), (rid, same)
        r = engine.requests[rid]
        assert r.prefill_count == 1 and r.decode_count == 15 and r.finished
    assert engine.runner.stats["graph_steps"] > 0        # decoding went through captured graphs
    assert engine.runner.stats["graph_deferred"] > 0     # after steps that were launched one by one
    assert engine.stats["queued_steps"] > 0              # and steps were queued behind the step that fed them
    engine.cache.assert_invariants()
    assert not engine.cache.requests
    assert engine.cache.page_groups[0].allocator.free_pages == 64


def test_temperature_sampling_equals_plain_chain(folders):
    """Tiny B, portions of 48 tokens mixed with decoding, 24 steps at temperature 0.8, fixed seeds."""
    from mini_hisparse_b200 import Engine

    cfg, page = TINY["B"]
    pc, w = P.load_folder(folders["B"])
    model = load(folders["B"], "float32")
    engine = Engine(model, num_pages=32, page_size=page, max_requests=4, max_tokens_per_step=48)
    prompts = {str(n): random_tokens(cfg["vocab_size"], n, seed=n) for n in (1, 31, 100, 257)}
    for i, (rid, prompt) in enumerate(prompts.items()):
        engine.add_request(rid, prompt, max_new_tokens=24, temperature=0.8, seed=1234 + i)
    out = engine.run()
    for i, (rid, prompt) in enumerate(prompts.items()):
        history = list(prompt)
        for step, token in enumerate(out[rid]):
            logits = P.forward_logits(pc, w, history)[-1]
            want, margin = P.sample_temperature(logits, 0.8, 1234 + i, step)
            assert token == want or margin < 1e-4, (rid, step, token, want, margin)
            history.append(token)
        assert len(out[rid]) == 24
    assert len({tuple(v) for v in out.values()}) == 4


def test_temperature_sampling_in_bfloat16(folders):
    """The same chain with bfloat16 logits: a token is the plain draw for the engine's own history,
    or the uniform number lies so close to an edge of that token's share of the CDF that the
    rounding of the logits decides; most draws are far from an edge and agree exactly."""
    from mini_hisparse_b200 import Engine

    cfg, page = TINY["B"]
    pc, w = P.load_folder(folders["B"])
    engine = Engine(load(folders["B"], "bfloat16"), num_pages=32, page_size=page, max_requests=4,
                    max_tokens_per_step=48)
    prompts = {str(n): random_tokens(cfg["vocab_size"], n, seed=n) for n in (1, 31, 100, 257)}
    for i, (rid, prompt) in enumerate(prompts.items()):
        engine.add_request(rid, prompt, max_new_tokens=24, temperature=0.8, seed=1234 + i)
    out = engine.run()
    exact = total = 0
    for i, (rid, prompt) in enumerate(prompts.items()):
        history = list(prompt)
        assert len(out[rid]) == 24
        for step, token in enumerate(out[rid]):
            logits = P.forward_logits(pc, w, history)[-1]
            want, _ = P.sample_temperature(logits, 0.8, 1234 + i, step)
            cdf = (logits.double() / 0.8).softmax(-1).cumsum(-1)
            u = P.uniform_from_counter(1234 + i, step) * float(cdf[-1])
            low, high = (float(cdf[token - 1]) if token else 0.0), float(cdf[token])
            assert max(low - u, u - high, 0.0) < 0.03, (rid, step, token, want)
            exact += token == want
            total += 1
            history.append(token)
    assert exact >= 0.85 * total, (exact, total)


def test_most_requests_in_one_step_on_the_engine(folders):
    """max_step_requests = 2 with four requests: steps hold two requests at most, everybody finishes,
    and the tokens are those of the plain implementation."""
    from mini_hisparse_b200 import Engine

    cfg, page = TINY["A"]
    pc, w = P.load_folder(folders["A"])
    engine = Engine(load(folders["A"], "float32"), num_pages=32, page_size=page, max_requests=4,
                    max_tokens_per_step=40, max_step_requests=2)
    prompts = {str(n): random_tokens(cfg["vocab_size"], n, seed=n) for n in (5, 21, 34, 9)}
    for rid, prompt in prompts.items():
        engine.add_request(rid, prompt, max_new_tokens=6)
    seen = 0
    while not engine.scheduler.idle or engine._queued is not None:
        engine.step()
        for held in list(engine.launch_log)[len(engine.launch_log) - (engine.launches - seen):]:
            assert 1 <= len(held) <= 2, held             # no step holds more than two requests
        seen = engine.launches
    assert all(t["tokens"] >= 1 for t in engine.timeline)
    for rid, prompt in prompts.items():
        assert engine.requests[rid].generated == P.generate(pc, w, prompt, 6)
    engine.cache.assert_invariants()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_observer_sees_every_layer(folders, dtype):
    """The observer hook of the step function: after every run entry it gets the residual stream and
    the entry's still-unadded output; their sum is the plain implementation's hidden state after
    that layer (the reference's hook: mini_hisparse/model.py:171-172, 202-203).  The prompt goes in
    two portions, so the second call of a layer sees rows of later positions."""
    from mini_hisparse_b200 import CacheConfig, CacheManager
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    cfg, page = TINY["B"]
    pc, w = P.load_folder(folders["B"])
    model = load(folders["B"], dtype)
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=8, page_size=page, max_requests=2,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    toks = random_tokens(cfg["vocab_size"], 50, seed=3)
    positions = torch.arange(50)
    x = w["model.embed_tokens.weight"].float()[torch.tensor(toks)]
    hidden = []
    for layer in range(cfg["num_hidden_layers"]):
        x = P.decoder_layer(pc, w, layer, x, positions)
        hidden.append(x)
    seen = []
    runner.observer = lambda i, residual, pending: seen.append(
        (i, (residual + pending.reduced()).float().cpu() if pending is not None else residual.float().cpu()))
    cache.open("a")
    runner.step([StepEntry("a", toks[:37], [])])
    runner.step([StepEntry("a", toks[37:], [12])])
    runner.check_status()
    layers = cfg["num_hidden_layers"]
    assert [i for i, _ in seen] == (list(range(layers)) + ["final"]) * 2
    for call, rows in ((0, slice(0, 37)), (1, slice(37, 50))):
        for layer in range(layers):
            got = seen[call * (layers + 1) + layer][1]
            ref = hidden[layer][rows]
            tol = dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=0.02 * float(ref.abs().max()), rtol=0.0)
            torch.testing.assert_close(got, ref, **tol)
        # after the last entry the hook gets the whole residual stream, the last output added
        torch.testing.assert_close(seen[call * (layers + 1) + layers][1], hidden[-1][rows], **tol)


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_long_decoding_and_first_tokens(folders, dtype):
    """A one-token prompt (positions 0, 1, 2, ... are all decoded) run far past several pages."""
    from mini_hisparse_b200 import Engine

    pc, w = P.load_folder(folders["A"])
    model = load(folders["A"], dtype)
    engine = Engine(model, num_pages=16, page_size=16, max_requests=2)
    engine.add_request("long", [5], max_new_tokens=200)
    out = engine.run()["long"]
    assert len(out) == 200
    logits = P.forward_logits(pc, w, [5] + out)
    picks = logits.argmax(-1)[:-1].tolist()
    if dtype == "float32":
        assert picks == out
    else:
        agree = sum(a == b for a, b in zip(picks, out)) / len(out)
        assert agree > 0.9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decoding_across_a_block_table_width_step(tmp_path, dtype):
    """A context that grows past 4,096 tokens (256 pages): the captured decode graph is keyed by the
    block table's width and has to be captured again at the step; the keys of a token are split
    over many CTAs.  Every decoded token must be the plain implementation's choice for the
    engine's own history (or lose to it by a near-tie in bfloat16)."""
    from mini_hisparse_b200 import Engine, write_random_model
    from conftest import TINY_A

    cfg = dict(TINY_A, max_position_embeddings=8192)
    write_random_model(cfg, 21, tmp_path, dtype=torch.bfloat16, matrix_std=0.1)
    pc, w = P.load_folder(tmp_path)
    model = load(tmp_path, dtype)
    prompt = random_tokens(cfg["vocab_size"], 4085, seed=5)
    engine = Engine(model, num_pages=300, page_size=16, max_requests=2, max_tokens_per_step=2048)
    engine.add_request("long", prompt, max_new_tokens=24)
    out = engine.run()["long"]
    assert len(out) == 24 and len(engine.runner.graphs) >= 2        # two widths were captured
    logits = P.forward_logits(pc, w, prompt + out)[len(prompt) - 1: -1]
    picks = logits.argmax(-1).tolist()
    if dtype == "float32":
        assert picks == out
    else:
        for i, (a, b) in enumerate(zip(out, picks)):
            gap = float(logits[i].max() - logits[i][a])
            assert a == b or gap < 0.05 * float(logits[i].abs().max()), (i, a, b, gap)


def test_few_pages_requests_wait_and_pages_are_used_again(folders):
    from mini_hisparse_b200 import CapacityError, Engine

    cfg, page = TINY["A"]
    pc, w = P.load_folder(folders["A"])
    model = load(folders["A"], "float32")
    # 6 pages of 16: one request of 40 + 8 tokens (3 pages) fits twice, never three times
    engine = Engine(model, num_pages=6, page_size=page, max_requests=4, max_tokens_per_step=64)
    prompts = {str(i): random_tokens(cfg["vocab_size"], 40, seed=i) for i in range(5)}
    for rid, p in prompts.items():
        engine.add_request(rid, p, max_new_tokens=8)
    with pytest.raises(CapacityError):
        engine.add_request("huge", [1] * 100, max_new_tokens=8)
    engine.step()
    assert len(engine.waiting) == 3 and len(engine.running) == 2
    out = engine.run()
    for rid, p in prompts.items():
        assert out[rid] == P.generate(pc, w, p, 8)
        assert engine.requests[rid].prefill_count == 1
    snap = engine.snapshot()
    assert snap["cache"]["page_groups"][0]["pages_reused"] > 0
    assert snap["scheduler"]["admissions_deferred"] > 0
    engine.cache.assert_invariants()


def test_cancel_and_eos(folders):
    from mini_hisparse_b200 import Engine

    cfg, page = TINY["A"]
    pc, w = P.load_folder(folders["A"])
    model = load(folders["A"], "float32")
    prompt = random_tokens(cfg["vocab_size"], 20, seed=3)
    want = P.generate(pc, w, prompt, 10)
    engine = Engine(model, num_pages=16, page_size=page, eos_token_id=want[4])
    engine.add_request("a", prompt, max_new_tokens=10)
    engine.add_request("b", prompt, max_new_tokens=10)
    engine.step()
    engine.cancel("b")
    out = engine.run()
    stop = want.index(want[4])
    assert out["a"] == want[: stop + 1]                   # the EOS token is kept
    assert engine.requests["b"].cancelled and not engine.cache.requests


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_queued_decode_steps_change_nothing(folders, dtype):
    """Decode steps queued behind the step that samples their input (token ids handed over on the
    device) against the same engine waiting for the host between steps: the same tokens, greedy and
    drawn at a temperature, with requests of different lengths and one that ends on an end token in
    the middle (found out one step late: one token is dropped).  In bfloat16 the step that still
    carries the ended request has other key splits than its counterpart, so there only the lengths
    and the end token are compared."""
    from mini_hisparse_b200 import Engine

    cfg, page = TINY["B"]
    model = load(folders["B"], dtype)
    prompts = {f"r{i}": random_tokens(cfg["vocab_size"], n, seed=40 + i) for i, n in enumerate((3, 50, 17, 90))}
    new_tokens, temperatures = (9, 30, 22, 14), (0.0, 0.7, 0.0, 1.1)

    def run(pipeline, eos):
        engine = Engine(model, num_pages=40, page_size=page, max_requests=5, max_tokens_per_step=64, pipeline=pipeline)
        for i, (rid, prompt) in enumerate(prompts.items()):
            engine.add_request(rid, prompt, max_new_tokens=new_tokens[i], temperature=temperatures[i], seed=7 + i,
                               eos_token_id=eos)
        out = engine.run()
        engine.cache.assert_invariants()
        assert not engine.cache.requests and engine._queued is None
        return out, engine.stats

    free_run, _ = run(False, None)
    eos = free_run["r1"][10]                     # r1's 11th token becomes everybody's end token
    waiting, stats0 = run(False, eos)
    queued, stats1 = run(True, eos)
    assert stats0["queued_steps"] == 0 and stats1["queued_steps"] > 5 and stats1["dropped_tokens"] >= 1
    assert waiting["r1"][-1] == eos and len(waiting["r1"]) <= 11
    if dtype == "float32":
        assert queued == waiting
    else:
        assert {k: len(v) for k, v in queued.items()} == {k: len(v) for k, v in waiting.items()}
        assert queued["r1"] == waiting["r1"]


def test_bad_weights_fail_with_one_clear_error(folders, tmp_path):
    from mini_hisparse_b200 import WeightError
    from mini_hisparse_b200.weights import write_safetensors

    w = P.read_safetensors(folders["B"] / "model.safetensors")
    del w["model.layers.2.mlp.up_proj.weight"]
    w["model.layers.0.self_attn.q_proj.bias"] = torch.zeros(7)
    w["model.layers.7.ghost"] = torch.zeros(2)
    bad = tmp_path / "bad"
    bad.mkdir()
    (bad / "config.json").write_text((folders["B"] / "config.json").read_text())
    write_safetensors(bad / "model.safetensors", w)
    with pytest.raises(WeightError) as e:
        load(bad, "float32")
    msg = str(e.value)
    assert "up_proj" in msg and "ghost" in msg and "q_proj.bias" in msg and "[7]" in msg


def test_command_line_generate(folders, tmp_path):
    out_file = tmp_path / "report.json"
    prompt = random_tokens(512, 9, seed=2)
    cmd = [sys.executable, "-m", "mini_hisparse_b200", "generate", "--model", str(folders["A"]),
           "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)), "--max-new-tokens", "6",
           "--gpu-pages", "8", "--output", str(out_file)]
    res = subprocess.run(cmd, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stderr[-2000:]
    report = json.loads(out_file.read_text())
    pc, w = P.load_folder(folders["A"])
    assert report["outputs"]["0"] == P.generate(pc, w, prompt, 6)
    assert report["requests"]["0"] == {"prefill_count": 1, "decode_count": 5, "generated_tokens": 6}
    assert json.loads(res.stdout)["outputs"] == report["outputs"]
