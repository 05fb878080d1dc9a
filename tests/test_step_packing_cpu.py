"""How a step's index arrays are packed, without a GPU: the batch's own arrays, one block table per
page group, and the arrays of every planner that the cache's users bring (the step function does
not know what they mean).  And what the engine does when a step raises."""
import numpy as np
import pytest
import torch

from mini_hisparse_b200.cache import CacheConfig, CacheManager
from mini_hisparse_b200.engine.step import BatchBuilder, StepEntry, StepError
from mini_hisparse_b200.parts import PartSpec, StepPlanner
from mini_hisparse_b200.parts.attention import ITEM_INTS, GQAttention
from mini_hisparse_b200.parts.spec import PagedKVNeed, PagedNeed, StateNeed
from dataclasses import dataclass


class CountingPlanner(StepPlanner):
    """A planner of a made-up mixer: one word per segment (its first position) and a running index."""

    def capacity(self, max_tokens, max_segments, fixed=None):
        return {"seg_first": max_segments, "tok_index": max_tokens + 3}

    def plan(self, segments, T, fixed=None):
        return ({"seg_first": np.asarray([s.start for s in segments], np.int32),
                 "tok_index": np.arange(T, dtype=np.int32)}, {"count": len(segments)})


class MadeUpMixer:
    def __init__(self, key):
        self.key = key

    def plan_key(self):
        return self.key

    def planner(self, page_size, sm_count):
        return CountingPlanner()


@dataclass(frozen=True)
class LatentNeed(PagedNeed):
    """A paged need with a page shape of its own: one vector of ``width`` per position."""

    width: int = 8
    window: int | None = None

    def page_shape(self, page_size):
        return (page_size, self.width)


def attention(nq, nkv, d=16):
    return GQAttention(PartSpec.make("gq_attention", hidden_size=32, q_heads=nq, kv_heads=nkv, head_dim=d,
                                     position=PartSpec.make("none")))


def test_packing_with_several_groups_and_planners():
    a4, a8 = attention(4, 2), attention(8, 2)          # same keys and values, other query heads
    needs = [a4.cache_need(), a8.cache_need(), LatentNeed(width=8), StateNeed((5,)), None]
    cache = CacheManager(needs, CacheConfig(num_pages=20, page_size=4, max_requests=3, dtype=torch.float32,
                                            device="cpu", allocate_storage=False))
    # equal needs share a pool and a block table whatever their query heads; the latent pages are a group of their own
    assert len(cache.page_groups) == 2 and len(cache.state_groups) == 1
    assert cache.page_groups[0].entries == [0, 1] and cache.page_groups[0].page_shape == (2, 2, 4, 16)
    assert cache.page_groups[1].page_shape == (4, 8) and cache.page_groups[1].page_bytes() == 4 * 8 * 4
    batch = BatchBuilder(cache, "cpu", sm_count=8)
    users = [batch.add_user(0, a4), batch.add_user(1, a8), batch.add_user(0, a4), batch.add_user(2, MadeUpMixer("m")),
             batch.add_user(3, MadeUpMixer("m")), batch.add_user(4, None)]
    # plans: one per (group, plan key): a4 (twice the same), a8, the made-up one; the state entry and None plan nothing
    assert len(batch.slots) == 3 and [batch.users[u][1] for u in users] == [0, 1, 0, 2, None, None]
    for name in ("x", "y"):
        cache.open(name)
    cache.ensure("x", 9), cache.advance("x", 9)
    entries = [StepEntry("x", [5, 6, 7], [0, 2]), StepEntry("y", [1, 2, 3, 4, 5, 6], [5])]
    segments, T = batch.segments(entries)
    assert T == 9 and [(s.start, s.count, s.offset) for s in segments] == [(9, 3, 0), (0, 6, 3)]
    for s in segments:
        cache.ensure(s.request, s.start + s.count)
    views = batch.eager(entries, segments)
    assert views["tokens"].tolist() == [5, 6, 7, 1, 2, 3, 4, 5, 6]
    assert views["positions"].tolist() == [9, 10, 11, 0, 1, 2, 3, 4, 5]
    assert views["tok_seg"].tolist() == [0, 0, 0, 1, 1, 1, 1, 1, 1]
    assert views["rows"].tolist() == [0, 2, 8]
    for gi, g in enumerate(cache.page_groups):
        table = views["tables"][gi]
        assert table.shape == (2, 3)                                   # 12 positions of 4 per page
        assert table[0].tolist() == g.tables[cache.slot("x")].pages
        assert table[1].tolist() == g.tables[cache.slot("y")].pages + [-1]
    v4, v8, vm = (batch.cache_view(u, views) for u in (users[0], users[1], users[3]))
    assert v4.meta["block_table"] is not None and v4.meta["n_small"] + v4.meta["n_big"] >= 2
    items4 = v4.meta["items"].view(-1, ITEM_INTS)[: v4.meta["n_small"] + v4.meta["n_big"]]
    items8 = v8.meta["items"].view(-1, ITEM_INTS)[: v8.meta["n_small"] + v8.meta["n_big"]]
    assert int(items4[:, 4].max()) == 2 and int(items8[:, 4].max()) == 4   # heads per KV group differ
    assert batch.cache_view(users[2], views).meta["items"].data_ptr() == v4.meta["items"].data_ptr()
    assert vm.meta["seg_first"].tolist() == [9, 0] and vm.meta["count"] == 2
    assert vm.meta["tok_index"].tolist() == list(range(9)) + [0, 0, 0]      # the rest of its capacity is zeroed
    assert vm.storage is None and vm.page_size == 4
    assert batch.cache_view(users[4], views).meta == {} and batch.cache_view(users[5], views) is None


def test_a_plan_larger_than_its_capacity_is_refused():
    class Liar(CountingPlanner):
        def capacity(self, max_tokens, max_segments, fixed=None):
            return {"seg_first": 0, "tok_index": max_tokens}

    class LiarMixer(MadeUpMixer):
        def planner(self, page_size, sm_count):
            return Liar()

    cache = CacheManager([LatentNeed()], CacheConfig(num_pages=4, page_size=4, max_requests=2, dtype=torch.float32,
                                                     device="cpu", allocate_storage=False))
    batch = BatchBuilder(cache, "cpu", sm_count=8)
    batch.add_user(0, LiarMixer("l"))
    cache.open("x")
    entries = [StepEntry("x", [1, 2], [])]
    segments, _ = batch.segments(entries)
    cache.ensure("x", 2)
    with pytest.raises(StepError, match="seg_first"):
        batch.eager(entries, segments)


def test_engine_fails_the_requests_of_a_step_that_raised():
    """Engine.step with a runner whose status check raises: the step's requests end as failed, their
    pages come back, the runner is told to put its scratch back, and the next step serves the rest."""
    from mini_hisparse_b200.engine.engine import Engine
    from mini_hisparse_b200.engine.scheduler import Scheduler, SchedulerConfig

    cache = CacheManager([PagedKVNeed(2, 16)], CacheConfig(num_pages=16, page_size=4, max_requests=4,
                                                           dtype=torch.float32, device="cpu", allocate_storage=False))

    class FakeRunner:
        def __init__(self):
            self.fail_next = False
            self.resets = 0
            self.stats = {}
            self.device_tokens_seen = 0

        use_graphs = True

        def step(self, entries, device_tokens=None):
            self.device_tokens_seen += device_tokens is not None
            for e in entries:                  # what the real runner does before and after its launches
                cache.ensure(e.request, cache.length(e.request) + len(e.tokens))
                cache.advance(e.request, len(e.tokens))
            return torch.zeros(sum(len(e.want) for e in entries), 50) if any(e.want for e in entries) else None

        def queue_status(self):
            pass

        def prepare_decode_ahead(self, requests):
            pass

        def check_status(self, queued=False):
            if self.fail_next:
                self.fail_next = False
                raise StepError("a bounded wait in the tensor-core matrix product ran out")

        def reset_after_error(self):
            self.resets += 1

    class FakeSampler:
        """Tickets as the real one; request i's k-th token is 10 i + k (from the counter it is given)."""

        def __init__(self):
            self.rows = {}
            self.ticket = 0

        def launch(self, logits, temps, seeds, counters):
            self.ticket += 1
            self.rows[self.ticket] = [3 + c for c in counters]
            return self.ticket

        def device_tokens(self, ticket):
            return torch.tensor(self.rows[ticket], dtype=torch.int32)

        def reset(self):
            self.rows.clear()

        def collect(self, ticket):
            return self.rows.pop(ticket)

    def make_engine(pipeline):
        from collections import deque

        engine = object.__new__(Engine)
        engine.cache, engine.runner, engine.sampler, engine.timeline = cache, FakeRunner(), FakeSampler(), []
        engine.scheduler = Scheduler(cache, SchedulerConfig(max_tokens_per_step=6), 50, eos_token_id=6)
        engine.pipeline, engine._queued, engine.launch_log, engine.launches = pipeline, None, deque(maxlen=8), 0
        engine.stats = {"queued_steps": 0, "dropped_tokens": 0}
        engine.model = None
        return engine

    engine = make_engine(pipeline=False)
    engine.add_request("a", [1, 2, 3], max_new_tokens=3)
    engine.add_request("b", [4, 5], max_new_tokens=3)
    engine.add_request("c", [6, 7, 8, 9], max_new_tokens=2)
    assert [t for _, t in engine.step()] == [3, 3]          # a and b whole, the first token of c
    engine.runner.fail_next = True
    with pytest.raises(StepError, match="bounded wait"):
        engine.step()                                       # a, b decode, c prefills: all three fail
    assert engine.runner.resets == 1
    assert all(engine.requests[n].failed for n in "abc") and not cache.requests
    cache.assert_invariants()
    assert cache.snapshot()["page_groups"][0]["pages_free"] == 16
    engine.add_request("d", [1, 2], max_new_tokens=2)       # the engine goes on
    assert engine.run()["d"] == [3, 4]

    # Decode steps queued behind one another: a step's tokens reach the host's books one call later,
    # every call returns one step's tokens, and a request that draws its end token (6 = 3 + 3) while
    # the next step is already queued costs one dropped token and no more.
    engine = make_engine(pipeline=True)
    engine.add_request("x", [1, 2], max_new_tokens=8)
    engine.add_request("y", [4], max_new_tokens=5)
    out = []
    while not engine.scheduler.idle or engine._queued is not None:
        out.append(engine.step())
    assert engine.requests["x"].generated == [3, 4, 5, 6]        # ended by its end token, kept
    assert engine.requests["y"].generated == [3, 4, 5, 6]
    assert [len(o) for o in out[:4]] == [2, 2, 2, 2] and all(len(o) == 0 for o in out[4:])
    assert engine.stats["queued_steps"] >= 2 and engine.stats["dropped_tokens"] == 2
    assert engine.runner.device_tokens_seen == engine.stats["queued_steps"]
    assert not cache.requests
    cache.assert_invariants()
    assert cache.snapshot()["page_groups"][0]["pages_free"] == 16


def test_status_bits_have_messages():
    """Every bit a kernel can set has a text, several bits give several texts, unknown bits are named."""
    from mini_hisparse_b200.engine.step import ModelRunner

    for bit, text in ModelRunner.STATUS_BITS.items():
        assert ModelRunner.status_message(bit) == text
    both = ModelRunner.status_message(4 | 8)
    assert "matrix product" in both and "TMA-fed attention" in both
    assert "0x40" in ModelRunner.status_message(64 | 1) and "vocabulary" in ModelRunner.status_message(64 | 1)
