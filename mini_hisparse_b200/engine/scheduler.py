"""The scheduler: admission, prompt portions under a token budget, decoding, finishing.

The reference admits at most one prompt per step, prefills it whole, then gives every running
request one sequential decode (mini_hisparse/engine.py:79-129).  It reserves a request's whole
lifetime of pages at admission (engine.py:53-55, 91-95), so a running request never runs out:
when pages are short, new requests WAIT (tests/test_engine.py:57-77) and nothing is preempted
or prefilled twice.  This scheduler keeps that policy and batches: every decoding request puts
one token into the step, and the rest of the step's token budget is cut from the prompts of
admitted requests in arrival order, so a long prompt is fed in portions beside the decodes.

The scheduler decides on the host only; it never touches the device, so its decisions are
tested without a GPU.
"""
from __future__ import annotations

from collections import deque
from dataclasses import dataclass, field

from ..cache.allocator import CapacityError
from ..sampling.sampler import SamplingParams


@dataclass
class Request:
    """mini_hisparse/engine.py:12-21, with portion counters instead of one prefill count."""

    request_id: object
    prompt: list[int]
    params: SamplingParams
    generated: list[int] = field(default_factory=list)
    prefilled: int = 0                 # prompt tokens already in the cache
    prefill_chunks: int = 0
    decode_count: int = 0
    admitted: bool = False
    finished: bool = False
    cancelled: bool = False
    failed: bool = False               # its step raised: what it holds was given back, it will not go on

    @property
    def max_new_tokens(self) -> int:
        return self.params.max_new_tokens

    @property
    def prefill_count(self) -> int:
        """1 once the whole prompt went through: prompts are never prefilled twice."""
        return 1 if self.prefilled >= len(self.prompt) else 0

    @property
    def decoding(self) -> bool:
        return self.admitted and not self.finished and self.prefilled >= len(self.prompt)


@dataclass
class Planned:
    request: Request
    tokens: list[int]
    sample: bool          # the last of these tokens yields the request's next token
    kind: str             # "prefill" or "decode"


@dataclass
class SchedulerConfig:
    max_tokens_per_step: int = 2048
    max_step_requests: int | None = None   # most requests in one step; None: all live ones

    def __post_init__(self):
        if self.max_tokens_per_step < 1:
            raise ValueError("max_tokens_per_step must be positive")


class Scheduler:
    def __init__(self, cache, config: SchedulerConfig, vocab_size: int,
                 max_positions: int | None = None, eos_token_id: int | None = None):
        self.cache, self.config = cache, config
        self.vocab_size, self.max_positions = vocab_size, max_positions
        self.eos_token_id = eos_token_id
        self.requests: dict[object, Request] = {}
        self.waiting: deque[Request] = deque()
        self.running: deque[Request] = deque()     # admitted and not finished, arrival order
        self.stats = {"steps": 0, "prefill_tokens": 0, "decode_tokens": 0, "admissions_deferred": 0}

    # ---- adding ------------------------------------------------------------------------------
    def add(self, request_id, prompt, params: SamplingParams) -> Request:
        """Validation of mini_hisparse/engine.py:48-65: unique id, non-empty prompt, ids inside the
        vocabulary, and a lifetime that an empty pool could hold."""
        prompt = list(prompt)
        if request_id in self.requests:
            raise ValueError(f"request id {request_id!r} is already in use")
        if not prompt:
            raise ValueError("the prompt cannot be empty")
        bad = [t for t in prompt if not 0 <= t < self.vocab_size]
        if bad:
            raise ValueError(f"token {bad[0]} is outside the model's vocabulary of {self.vocab_size}")
        total = len(prompt) + params.max_new_tokens
        if self.max_positions is not None and total > self.max_positions:
            raise ValueError(
                f"prompt ({len(prompt)}) plus max_new_tokens ({params.max_new_tokens}) exceeds "
                f"max_position_embeddings ({self.max_positions})"
            )
        if not self.cache.can_ever_fit(total, self.config.max_tokens_per_step):
            raise CapacityError("the request cannot fit even in an empty page pool")
        request = Request(request_id, prompt, params)
        self.requests[request_id] = request
        self.waiting.append(request)
        return request

    # ---- planning a step ----------------------------------------------------------------------
    def plan(self) -> list[Planned]:
        budget = self.config.max_tokens_per_step
        cap = self.config.max_step_requests
        planned: list[Planned] = []
        # 1. one token for every decoding request; if the budget is smaller than their number, the
        #    deque rotates so that nobody starves
        decoders = [r for r in self.running if r.decoding]
        take = min(len(decoders), budget, cap if cap is not None else len(decoders))
        for r in decoders[:take]:
            planned.append(Planned(r, [r.generated[-1]], True, "decode"))
        budget -= take
        if take < len(decoders):
            for r in decoders[:take]:
                self.running.remove(r)
                self.running.append(r)
        # 2. admit from the head of the queue while credits, slots and budget last (arrival order)
        prefilling = [r for r in self.running if not r.decoding]
        pending_budget = budget - sum(len(r.prompt) - r.prefilled for r in prefilling)
        while self.waiting and pending_budget > 0:
            head = self.waiting[0]
            try:
                self.cache.open(head.request_id, reserve_tokens=len(head.prompt) + head.max_new_tokens,
                                max_step_tokens=self.config.max_tokens_per_step)
            except CapacityError:
                if not self.running:
                    raise      # nothing will ever free pages for it
                self.stats["admissions_deferred"] += 1
                break
            self.waiting.popleft()
            head.admitted = True
            self.running.append(head)
            prefilling.append(head)
            pending_budget -= len(head.prompt)
        # 3. portions of prompts, oldest first
        for r in prefilling:
            if budget <= 0 or (cap is not None and len(planned) >= cap):
                break
            n = min(len(r.prompt) - r.prefilled, budget)
            tokens = r.prompt[r.prefilled : r.prefilled + n]
            last = r.prefilled + n == len(r.prompt)
            planned.append(Planned(r, tokens, last, "prefill"))
            budget -= n
        return planned

    # ---- after the step --------------------------------------------------------------------------
    def commit(self, planned: list[Planned], sampled: list[int]) -> list[tuple[object, int]]:
        """``sampled`` holds one token for every planned entry with sample=True, in order."""
        emitted = []
        it = iter(sampled)
        for p in planned:
            r = p.request
            if p.kind == "prefill":
                r.prefilled += len(p.tokens)
                r.prefill_chunks += 1
                self.stats["prefill_tokens"] += len(p.tokens)
            else:
                r.decode_count += 1
                self.stats["decode_tokens"] += 1
            if not p.sample:
                continue
            token = next(it)
            if r.finished:          # cancelled while the step ran
                continue
            r.generated.append(token)
            emitted.append((r.request_id, token))
            eos = r.params.eos_token_id if r.params.eos_token_id is not None else self.eos_token_id
            if token == eos or len(r.generated) >= r.max_new_tokens:
                self._finish(r)
        self.stats["steps"] += 1
        return emitted

    def _finish(self, r: Request) -> None:
        """mini_hisparse/engine.py:74-76: mark finished and give everything back at once."""
        r.finished = True
        if r in self.running:
            self.running.remove(r)
        if r.admitted:
            self.cache.close(r.request_id)

    def cancel(self, request_id) -> None:
        """mini_hisparse/engine.py:137-146: drop a waiting request, or release a running one."""
        r = self.requests[request_id]
        if r.finished:
            return
        if r in self.waiting:
            self.waiting.remove(r)
            r.finished = r.cancelled = True
            return
        r.cancelled = True
        self._finish(r)

    def fail(self, planned: list[Planned]) -> list[object]:
        """The step that ran ``planned`` raised after the cache may already have taken its tokens:
        the requests' positions in the cache and in the scheduler's books no longer agree, so none
        of them can go on.  Each is finished as failed and gives back what it holds; requests that
        were not in the step are untouched.  Returns the failed ids."""
        failed = []
        for p in planned:
            r = p.request
            if r.finished:
                continue
            r.failed = True
            self._finish(r)
            failed.append(r.request_id)
        self.stats["failed_requests"] = self.stats.get("failed_requests", 0) + len(failed)
        return failed

    @property
    def idle(self) -> bool:
        return not self.waiting and not self.running
