"""Replay through bin/trace_run: the same requests whole, with the last 32 tokens one by one (three
requests side by side, through the captured decode graphs and the steps packed ahead), in portions
of changing size, and mixed with other requests in a pool so small that pages are used again, in
float32 and in bfloat16.  Every logit row is compared with the plain implementation; the
bfloat16 rows also with the engine's own float32 run of the same cut.  Pages that are given back
are overwritten (--poison), so a read of a stale page cannot pass."""
import pytest
import torch

import schedules
from conftest import BF16_BOUNDS, TINY, TraceRun, random_tokens, row_rms_error, tolerances
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

LENGTHS = {"A": [7, 33, 64, 100, 129, 50], "B": [1, 31, 100, 257, 64, 18], "C": [40, 150, 9, 280, 3, 65],
           "D": [70, 5, 200, 33, 64, 2], "E": [90, 3, 170, 48, 25, 131], "F": [30, 61, 8, 100, 2, 49]}

MODES = {
    "whole": schedules.whole,
    "tail_one_by_one": schedules.tail_one_by_one,
    "changing_portions": schedules.changing_portions,
    "mixed": schedules.mixed,
}


def requests_of(name):
    vocab = TINY[name][0]["vocab_size"]
    return {f"r{i}": random_tokens(vocab, n, seed=100 + i) for i, n in enumerate(LENGTHS[name])}


def plans_of(name):
    requests = requests_of(name)
    return {mode: fn(requests) for mode, fn in MODES.items()}


@pytest.fixture(scope="module")
def plain_logits(folders):
    """(name, act) -> {request: logits of every position} of the plain implementation; act = None, or
    torch.bfloat16 for the run whose activations between the parts are rounded as the engine's are."""
    cache = {}

    def get(name, act=None):
        if (name, act) not in cache:
            cfg, w = P.load_folder(folders[name])
            cache[(name, act)] = {rid: P.forward_logits(cfg, w, toks, act=act)
                                  for rid, toks in requests_of(name).items()}
        return cache[(name, act)]

    return get


@pytest.fixture(scope="module")
def replayed(folders, tmp_path_factory):
    """(name, dtype) -> {mode: [logits of each step]} and the program's counters, replayed once."""
    cache = {}

    def get(name, dtype):
        if (name, dtype) in cache:
            return cache[(name, dtype)]
        page = TINY[name][1]
        plans = plans_of(name)
        # the pool is as small as the fullest moment of any mode needs: pages are used again
        max_tokens = max(schedules.peak_tokens(steps, round_to=max(64, page)) for steps in plans.values())
        run = TraceRun(folders[name], dtype, tmp_path_factory.mktemp(f"replay{name}{dtype}"), max_tokens,
                       page_size=page, extra=("--poison",))
        try:
            out = {mode: [run.step(entries, end) for entries, end in steps] for mode, steps in plans.items()}
            assert run.close() == 0
        finally:
            if run.proc.poll() is None:
                run.proc.kill()
        cache[(name, dtype)] = (out, run.stats())
        return cache[(name, dtype)]

    return get


def compare(name, mode, steps, logits, reference_rows, tol_of, what):
    """Every row of every step against ``reference_rows(request, first, count)``; returns the worst
    error as a share of the request's largest reference logit, and how many top-1 choices agree."""
    done = {}
    worst, rms, same, rows_seen = 0.0, 0.0, 0, 0
    page = TINY[name][1]
    for (entries, end), got_all in zip(steps, logits):
        row = 0
        for e in entries:
            rid, n = e["id"], len(e["tokens"])
            first = done.get(rid, 0)
            ref, ref_all = reference_rows(rid, first, n)
            got = got_all[row: row + n]
            worst = max(worst, float((got - ref).abs().max()) / float(ref_all.abs().max()))
            rms = max(rms, row_rms_error(got, ref))
            try:
                torch.testing.assert_close(got, ref, **tol_of(ref_all))
            except AssertionError as err:
                bad = (got - ref).abs().amax(-1)
                first_bad = int((bad > bad.max() * 0.5).nonzero()[0])
                raise AssertionError(
                    f"{name} {mode} vs {what}: request {rid} first wrong token at position {first + first_bad} "
                    f"(portion of {n} starting at {first}, page size {page}): {err}") from None
            same += int((got.argmax(-1) == ref.argmax(-1)).sum())
            rows_seen += n
            row += n
            done[rid] = first + n
    return worst, rms, same, rows_seen, done


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", list(TINY))
def test_replay_all_cuts(plain_logits, replayed, name, dtype):
    requests = requests_of(name)
    plans = plans_of(name)
    out, stats = replayed(name, dtype)
    plain = plain_logits(name)
    for mode, steps in plans.items():
        worst, rms, same, rows_seen, done = compare(
            name, mode, steps, out[mode], lambda rid, a, n: (plain[rid][a: a + n], plain[rid]),
            lambda ref: tolerances(dtype, ref, name), "the plain implementation")
        assert all(done[rid] == len(t) for rid, t in requests.items()), mode
        print(f"replay {name} {dtype} {mode}: worst error {worst:.2e} of the largest logit, worst row rms "
              f"{rms:.2e} of the row's, top-1 agrees on {same} of {rows_seen} rows")
        assert dtype == "float32" or rms < BF16_BOUNDS[name][1], (mode, rms)
        # float32 picks the same token everywhere (bar one exact tie); bfloat16 may flip near-ties
        assert same >= (rows_seen - 1 if dtype == "float32" else 0.9 * rows_seen), (mode, same, rows_seen)
    if dtype == "bfloat16":
        # the plain implementation with its activations rounded to bfloat16 where the engine rounds its
        # own (sums stay float32): what is left is the order of the sums and the places where a rounding
        # fell the other way, a fraction of what bfloat16 itself costs
        rounded = plain_logits(name, torch.bfloat16)
        for mode, steps in plans.items():
            worst, rms, *_ = compare(name, mode, steps, out[mode],
                                     lambda rid, a, n: (rounded[rid][a: a + n], rounded[rid]),
                                     lambda ref: tolerances(dtype, ref, name),
                                     "the plain implementation with bfloat16 activations")
            print(f"replay {name} bfloat16 {mode}: worst error {worst:.2e}, worst row rms {rms:.2e} against the "
                  f"plain implementation with bfloat16 activations")
        # the same cut in the engine's own float32: what is left is the rounding of activations alone
        own, _ = replayed(name, "float32")
        for mode, steps in plans.items():
            flat = {}
            for (entries, end), rows in zip(steps, own[mode]):
                row = 0
                for e in entries:
                    flat.setdefault(e["id"], []).append(rows[row: row + len(e["tokens"])])
                    row += len(e["tokens"])
            own_rows = {rid: torch.cat(parts) for rid, parts in flat.items()}
            worst, rms, *_ = compare(name, mode, steps, out[mode],
                                lambda rid, a, n: (own_rows[rid][a: a + n], own_rows[rid]),
                                lambda ref: tolerances(dtype, ref, name),
                                "the engine's float32 run")
            print(f"replay {name} bfloat16 {mode}: worst error {worst:.2e}, worst row rms {rms:.2e} against the "
                  f"engine's own float32 run")
            assert rms < BF16_BOUNDS[name][1], (mode, rms)
    # the decode steps went through captured graphs, several requests at a time, and some were packed ahead
    runner, cache = stats["runner"], stats["cache"]
    assert runner["graph_steps"] >= 32 and runner["graph_captures"] >= 2, runner
    assert runner["prepared_steps"] > 0, runner
    assert cache["page_groups"][0]["pages_reused"] > 0 and cache["page_groups"][0]["pages_poisoned"] > 0, cache
    if name == "C":
        # its longest request decodes across position 256: the decode graph's block table doubles
        assert runner["graph_captures"] >= 3, runner


def test_replay_without_graphs_gives_the_same_rows(folders, replayed, tmp_path):
    """--no-graphs launches the same decode steps eagerly (other key splits): float32 rows agree to
    rounding with the captured ones."""
    name = "A"
    steps = plans_of(name)["tail_one_by_one"]
    out, _ = replayed(name, "float32")
    run = TraceRun(folders[name], "float32", tmp_path / "o", schedules.peak_tokens(steps), page_size=TINY[name][1],
                   extra=("--no-graphs",))
    try:
        for (entries, end), want in zip(steps, out["tail_one_by_one"]):
            torch.testing.assert_close(run.step(entries, end), want, atol=3e-5, rtol=3e-5)
        assert run.close() == 0
        assert run.stats()["runner"]["graph_steps"] == 0
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
