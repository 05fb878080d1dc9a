"""Replay through bin/trace_run: the same requests whole, with the last 32 tokens one by one, in
portions of changing size, and mixed with other requests in a pool so small that pages are used
again, in float32 and in bfloat16; every logit row is compared with the plain implementation."""
import pytest
import torch

import schedules
from conftest import TINY, TraceRun, random_tokens, tolerances
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [7, 33, 64, 100, 129, 50], "B": [1, 31, 100, 257, 64, 18], "C": [40, 150, 9, 77, 3, 65],
           "D": [70, 5, 200, 33, 64, 2]}


def requests_of(name):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}


@pytest.fixture(scope="module")
def plain_logits(folders):
    out = {}
    for name in TINY:
        cfg, w = P.load_folder(folders[name])
        out[name] = {rid: P.forward_logits(cfg, w, toks) for rid, toks in requests_of(name).items()}
    return out


MODES = {
    "whole": schedules.whole,
    "tail_one_by_one": schedules.tail_one_by_one,
    "changing_portions": schedules.changing_portions,
    "mixed": schedules.mixed,
}


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C", "D"])
def test_replay_all_cuts(folders, plain_logits, tmp_path, name, dtype):
    requests = requests_of(name)
    page = TINY[name][1]
    plans = {mode: fn(requests) for mode, fn in MODES.items()}
    # the pool is as small as the fullest moment of any mode needs: pages are used again
    max_tokens = max(schedules.peak_tokens(steps) for steps in plans.values())
    run = TraceRun(folders[name], dtype, tmp_path / "out", max_tokens, page_size=page)
    try:
        for mode, steps in plans.items():
            done = {rid: 0 for rid in requests}
            worst = 0.0
            same = rows_seen = 0
            for entries, end in steps:
                logits = run.step(entries, end)
                row = 0
                for e in entries:
                    n = len(e["tokens"])
                    ref = plain_logits[name][e["id"]][done[e["id"]]: done[e["id"]] + n]
                    got = logits[row: row + n]
                    worst = max(worst, float((got - ref).abs().max()))
                    try:
                        torch.testing.assert_close(got, ref, **tolerances(dtype, plain_logits[name][e["id"]]))
                    except AssertionError as err:
                        bad = (got - ref).abs().amax(-1)
                        first = int((bad > bad.max() * 0.5).nonzero()[0])
                        raise AssertionError(
                            f"{mode}: request {e['id']} first wrong token at position "
                            f"{done[e['id']] + first} (portion of {n} starting at {done[e['id']]}, "
                            f"page size {page}): {err}") from None
                    same += int((got.argmax(-1) == ref.argmax(-1)).sum())
                    rows_seen += n
                    row += n
                    done[e["id"]] += n
            assert all(done[rid] == len(t) for rid, t in requests.items()), mode
            # bfloat16 may flip near-ties of the top logit; over a whole mode nine in ten must agree
            assert same >= (1.0 if dtype == "float32" else 0.9) * rows_seen - (1 if dtype == "float32" else 0), (mode, same, rows_seen)
        assert run.close() == 0
    finally:
        if run.proc.poll() is None:
            run.proc.kill()


def test_trace_run_wants_nothing_writes_nothing(folders, tmp_path):
    toks = random_tokens(512, 20, 1)
    run = TraceRun(folders["A"], "float32", tmp_path / "o", 64)
    assert run.step([{"id": "a", "tokens": toks[:10], "want": []}]) is None
    got = run.step([{"id": "a", "tokens": toks[10:], "want": [9]}], end=["a"])
    assert got.shape == (1, 512)
    cfg, w = P.load_folder(folders["A"])
    torch.testing.assert_close(got[0], P.forward_logits(cfg, w, toks)[-1], atol=3e-5, rtol=3e-5)
    assert run.close() == 0
