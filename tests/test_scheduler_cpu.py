"""The scheduler's decisions, without a GPU: a fake step stands in for the model."""
import pytest
import torch

from mini_hisparse_b200.cache import CacheConfig, CacheManager, CapacityError
from mini_hisparse_b200.engine.scheduler import Scheduler, SchedulerConfig
from mini_hisparse_b200.parts.spec import PagedKVNeed
from mini_hisparse_b200.sampling import SamplingParams


def make(num_pages=16, page_size=4, max_requests=4, budget=8, vocab=50, max_positions=None, eos=None):
    cache = CacheManager([PagedKVNeed(2, 16)] * 2,
                         CacheConfig(num_pages=num_pages, page_size=page_size, max_requests=max_requests,
                                     dtype=torch.float32, device="cpu", allocate_storage=False))
    return Scheduler(cache, SchedulerConfig(max_tokens_per_step=budget), vocab, max_positions, eos), cache


def fake_step(sched, cache, planned, token=lambda r: 7):
    """What the engine does around the model: grow the cache, 'sample', commit."""
    for p in planned:
        rid = p.request.request_id
        cache.ensure(rid, cache.length(rid) + len(p.tokens))
        cache.advance(rid, len(p.tokens))
    cache.assert_invariants()
    return sched.commit(planned, [token(p.request) for p in planned if p.sample])


def test_validation_at_add():
    s, _ = make(max_positions=30)
    s.add("a", [1, 2, 3], SamplingParams(4))
    with pytest.raises(ValueError, match="already"):
        s.add("a", [1], SamplingParams(4))
    with pytest.raises(ValueError, match="empty"):
        s.add("b", [], SamplingParams(4))
    with pytest.raises(ValueError, match="vocabulary"):
        s.add("b", [1, 50], SamplingParams(4))
    with pytest.raises(ValueError, match="max_position"):
        s.add("b", [1] * 28, SamplingParams(4))
    with pytest.raises(ValueError):
        SamplingParams(0)
    s2, _ = make(num_pages=4)
    with pytest.raises(CapacityError, match="empty page pool"):
        s2.add("big", [1] * 14, SamplingParams(4))


def test_prompt_is_cut_into_portions_under_the_budget():
    s, c = make(budget=8)
    r = s.add("a", list(range(1, 22)), SamplingParams(3))
    sizes = []
    while not r.decoding:
        planned = s.plan()
        assert sum(len(p.tokens) for p in planned) <= 8
        sizes.append(len(planned[0].tokens))
        assert planned[0].sample == (r.prefilled + len(planned[0].tokens) == 21)
        fake_step(s, c, planned)
    assert sizes == [8, 8, 5] and r.prefill_chunks == 3 and r.prefill_count == 1
    assert r.generated == [7]                  # the last portion's last row gave the first token
    planned = s.plan()
    assert [(p.kind, p.tokens) for p in planned] == [("decode", [7])]


def test_decodes_go_first_and_prompts_fill_the_rest():
    s, c = make(budget=6, num_pages=32)
    a = s.add("a", [1, 2, 3], SamplingParams(10))
    fake_step(s, c, s.plan())
    assert a.decoding
    b = s.add("b", list(range(1, 12)), SamplingParams(2))
    planned = s.plan()
    assert [(p.request.request_id, p.kind, len(p.tokens)) for p in planned] == [("a", "decode", 1), ("b", "prefill", 5)]
    fake_step(s, c, planned)
    planned = s.plan()
    assert [(p.request.request_id, len(p.tokens), p.sample) for p in planned] == [("a", 1, True), ("b", 5, False)]
    fake_step(s, c, planned)
    planned = s.plan()
    assert [(p.request.request_id, len(p.tokens), p.sample) for p in planned] == [("a", 1, True), ("b", 1, True)]


def test_when_pages_run_out_new_requests_wait_and_nothing_is_prefilled_twice():
    # the pool holds one request's lifetime (10 + 5 tokens = 4 pages of 4); the others wait in order
    s, c = make(num_pages=4, budget=16)
    rs = [s.add(str(i), [1] * 10, SamplingParams(5)) for i in range(3)]
    fake_step(s, c, s.plan())
    assert len(s.waiting) == 2 and s.stats["admissions_deferred"] == 1
    order = []
    for _ in range(100):
        if s.idle:
            break
        planned = s.plan()
        for p in planned:
            if p.kind == "prefill" and p.request.prefilled == 0:
                order.append(p.request.request_id)
        fake_step(s, c, planned)
    assert s.idle and order == ["1", "2"]
    assert all(len(r.generated) == 5 and r.prefill_count == 1 and r.decode_count == 4 for r in rs)
    assert not c.requests and c.page_groups[0].allocator.free_pages == 4
    assert c.page_groups[0].allocator.reuses > 0


def test_finish_on_eos_and_length_and_cancel():
    s, c = make(eos=9, num_pages=32)
    a = s.add("a", [1, 2], SamplingParams(5))
    b = s.add("b", [3, 4], SamplingParams(2))
    w = s.add("w", [5], SamplingParams(5))
    fake_step(s, c, s.plan(), token=lambda r: 9 if r.request_id == "a" else 4)
    assert a.finished and a.generated == [9] and "a" not in c.requests      # the EOS token is kept
    fake_step(s, c, s.plan(), token=lambda r: 4)
    assert b.finished and b.generated == [4, 4] and b.decode_count == 1
    s.cancel("w")
    assert w.finished and w.cancelled and "w" not in c.requests
    late = s.add("late", [1, 2, 3], SamplingParams(2))
    s.cancel("late")                         # cancelled while still waiting: never admitted
    assert late.cancelled and not late.admitted and s.idle
    c.assert_invariants()
    assert c.page_groups[0].allocator.free_pages == 32


def test_cancel_in_the_middle_of_a_prompt():
    s, c = make(budget=4, num_pages=32)
    a = s.add("a", list(range(1, 14)), SamplingParams(3))
    fake_step(s, c, s.plan())
    assert 0 < a.prefilled < 13
    s.cancel("a")
    assert a.cancelled and s.idle and not c.requests
    c.assert_invariants()


def test_more_decoders_than_budget_take_turns():
    s, c = make(budget=8, num_pages=64, max_requests=4)
    rs = [s.add(str(i), [1], SamplingParams(6)) for i in range(3)]
    fake_step(s, c, s.plan())
    assert all(r.decoding for r in rs)
    s.config.max_tokens_per_step = 2
    seen = []
    for _ in range(6):
        planned = s.plan()
        assert len(planned) == 2
        seen += [p.request.request_id for p in planned]
        fake_step(s, c, planned)
    assert {seen.count(x) for x in "012"} == {4}


def test_most_requests_in_one_step():
    """max_step_requests caps how many requests share a step: the decoders take turns (the deque
    rotates, nobody starves) and a prompt waits for a free place."""
    cache = CacheManager([PagedKVNeed(2, 16)] * 2,
                         CacheConfig(num_pages=32, page_size=4, max_requests=6, dtype=torch.float32, device="cpu",
                                     allocate_storage=False))
    s = Scheduler(cache, SchedulerConfig(max_tokens_per_step=64, max_step_requests=2), 50)
    for name in "abc":
        s.add(name, [1, 2, 3], SamplingParams(6))
    turns = {n: 0 for n in "abcd"}
    late_added = False
    for step in range(40):
        if s.idle:
            break
        planned = s.plan()
        assert 1 <= len(planned) <= 2, [p.request.request_id for p in planned]
        for p in planned:
            turns[p.request.request_id] += 1
        fake_step(s, cache, planned)
        if step == 3 and not late_added:
            s.add("d", [4, 5, 6, 7], SamplingParams(2))     # a prompt that arrives while three decode
            late_added = True
    assert s.idle
    assert all(len(s.requests[n].generated) == 6 for n in "abc") and len(s.requests["d"].generated) == 2
    assert turns["a"] == turns["b"] == turns["c"] == 6      # one prompt step and five decode steps each
    cache.assert_invariants()
    assert cache.snapshot()["page_groups"][0]["pages_free"] == 32


def test_a_failed_step_finishes_its_requests_and_frees_their_pages():
    """A step raised after the cache had taken its tokens: its requests cannot be fed again (their
    cache positions ran ahead of the scheduler's books), so they end as failed and give everything
    back; a request that was not in the step goes on."""
    s, c = make(num_pages=16, budget=6)
    s.add("a", [1, 2, 3, 4], SamplingParams(4))
    s.add("b", [5, 6], SamplingParams(4))
    s.add("late", list(range(1, 9)), SamplingParams(2))
    planned = s.plan()                       # a whole, b whole, nothing of late (budget 6)
    assert [p.request.request_id for p in planned] == ["a", "b"]
    for p in planned:                        # the runner got as far as growing the cache, then raised
        rid = p.request.request_id
        c.ensure(rid, len(p.tokens))
        c.advance(rid, len(p.tokens))
    failed = s.fail(planned)
    assert failed == ["a", "b"]
    assert all(s.requests[n].failed and s.requests[n].finished and not s.requests[n].generated for n in "ab")
    assert "a" not in c.requests and "b" not in c.requests
    c.assert_invariants()
    assert c.snapshot()["page_groups"][0]["pages_free"] == 16
    while not s.idle:                        # the third request is served as if nothing had happened
        fake_step(s, c, s.plan())
    assert s.requests["late"].generated == [7, 7] and not s.requests["late"].failed
    assert s.stats["failed_requests"] == 2
