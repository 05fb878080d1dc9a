"""The Python entry point: load a model folder, add requests, step, run.

In the reference's manner (mini_hisparse/engine.py:24-146; examples/long_context_chat.py:58-81):
``Engine.add_request(request_id, prompt, max_new_tokens)``, ``step() -> [(id, token)]``,
``run() -> {id: tokens}``, ``cancel(id)``; ``load_model`` stands where
``MiniModel.from_pretrained(name, device, dtype)`` does (mini_hisparse/model.py:98-125).
"""
from __future__ import annotations

from collections import deque
from pathlib import Path

import torch

from ..cache.manager import CacheConfig, CacheManager
from ..config.registry import resolve
from ..models.decoder import DecoderModel
from ..parts.base import Runtime
from ..sampling.sampler import Sampler, SamplingParams
from ..weights.loader import init_random, load_weights
from .scheduler import Planned, Request, Scheduler, SchedulerConfig
from .step import ModelRunner, StepEntry, StepError

_DTYPES = {"float32": torch.float32, "bfloat16": torch.bfloat16, "fp32": torch.float32,
           "bf16": torch.bfloat16, torch.float32: torch.float32, torch.bfloat16: torch.bfloat16}


def parse_dtype(dtype) -> torch.dtype:
    try:
        return _DTYPES[dtype]
    except KeyError:
        raise ValueError(f"dtype must be float32 or bfloat16, not {dtype!r}") from None


def make_runtime(device="cuda:0", dtype="bfloat16") -> Runtime:
    from ..kernels.runtime import make_runtime as _make

    return _make(device, parse_dtype(dtype))


def load_model(source, device="cuda:0", dtype="bfloat16", random_seed: int | None = None) -> DecoderModel:
    """Build the model that ``source`` (a folder with config.json, a config file, or a config
    mapping) names in its "architectures", and load its safetensors weights; with
    ``random_seed`` the weights are drawn on the device instead and no file is read."""
    cfg, spec = resolve(source)
    rt = make_runtime(device, dtype)
    model = DecoderModel(spec, rt, config=cfg)
    if random_seed is not None:
        init_random(model, random_seed)
    else:
        load_weights(model, Path(source))
    return model


class Engine:
    def __init__(self, model: DecoderModel, cache_config: CacheConfig | None = None, *,
                 num_pages: int | None = None, page_size: int = 16, max_requests: int = 8,
                 max_tokens_per_step: int = 2048, eos_token_id: int | None = None,
                 use_graphs: bool = True, max_step_requests: int | None = None, pipeline: bool = True,
                 graph_after: int = 8):
        self.model = model
        if cache_config is None:
            if num_pages is None:
                raise ValueError("give a CacheConfig or num_pages")
            width = None
            if model.spec.max_positions:
                width = min(num_pages, -(-model.spec.max_positions // page_size))
            cache_config = CacheConfig(num_pages=num_pages, page_size=page_size,
                                       max_requests=max_requests, max_pages_per_request=width,
                                       dtype=model.rt.dtype, device=str(model.rt.device))
        if cache_config.dtype != model.rt.dtype or torch.device(cache_config.device) != model.rt.device:
            raise ValueError("model/cache dtype or device differ")   # mini_hisparse/engine.py:36-38
        self.cache = CacheManager(model.cache_needs, cache_config)
        # graph_after: a batch of decoding requests gets its captured graph at the graph_after-th step that
        # could use it; until then its steps are launched kernel by kernel (a capture costs several steps'
        # time, which a batch that changes every few steps never earns back)
        self.runner = ModelRunner(model, self.cache, use_graphs=use_graphs, graph_after=graph_after)
        eos = eos_token_id if eos_token_id is not None else model.spec.eos_token_id
        self.scheduler = Scheduler(self.cache, SchedulerConfig(max_tokens_per_step, max_step_requests),
                                   model.spec.vocab_size, model.spec.max_positions, eos)
        self.sampler = Sampler(model.rt.device, max_rows=cache_config.max_requests)
        self.timeline: list[dict] = []
        # what the last steps held, for whoever measures them: per launched step a list of
        # (request, cached positions before, new tokens); ``launches`` counts all of them
        self.launch_log: deque = deque(maxlen=64)
        self.launches = 0
        self.stats = {"queued_steps": 0, "dropped_tokens": 0}
        self.pipeline = pipeline        # queue a decode step behind the one that samples its input
        self._queued = None             # the step that was queued that way and is not collected yet

    # ---- the reference's five calls ------------------------------------------------------------
    @property
    def requests(self) -> dict:
        return self.scheduler.requests

    @property
    def waiting(self):
        return self.scheduler.waiting

    @property
    def running(self):
        return self.scheduler.running

    def add_request(self, request_id, prompt, max_new_tokens: int = 16, temperature: float = 0.0,
                    seed: int = 0, eos_token_id: int | None = None) -> Request:
        params = SamplingParams(max_new_tokens=max_new_tokens, temperature=temperature, seed=seed,
                                eos_token_id=eos_token_id)
        return self.scheduler.add(request_id, prompt, params)

    def step(self) -> list[tuple[object, int]]:
        """One scheduler tick: plan, run the batch, sample, commit; returns the step's (id, token) pairs.

        Decode steps overlap: while a step of single tokens runs, and if its requests will all want
        another token whatever this one turns out to be, the NEXT step is queued behind it with its
        token ids taken from the sampler's output on the device, and only then does the host wait for
        this step's tokens.  So the GPU goes from one step to the next without waiting for the host,
        and a call returns one step's tokens as before.  A request that ends on its end-of-sequence
        token is found out one step late: the step that was queued for it computes a token that is
        dropped, at positions its reservation covers, and its pages are given back in stream order.

        If a kernel reports a fault (StepError), every request of the steps in flight is finished as
        failed and gives back its pages (the cache had already taken their tokens, so they could not
        be fed again), the runner's self-resetting scratch is put back to zero, and the error is
        raised; the engine and the requests that were not in those steps go on."""
        current, self._queued = self._queued, None
        if current is None:
            planned = self.scheduler.plan()
            if not planned:
                return []
            current = self._launch(planned)
        try:
            following = self._following(current)
            if following is not None:
                self._queued = self._launch(following, behind=current)
            sampled = self._collect(current)
        except StepError:
            self.runner.reset_after_error()
            self.scheduler.fail(current["planned"])
            if self._queued is not None:
                self.scheduler.fail(self._queued["planned"])
                self._queued = None
            self.sampler.reset()
            raise
        self.stats["dropped_tokens"] += sum(1 for p in current["planned"] if p.sample and p.request.finished)
        emitted = self.scheduler.commit(current["planned"], sampled)
        if self._queued is not None:
            # the queued step ran on the device's copy of these tokens; the host's books get them now
            tokens = dict(emitted)
            for p in self._queued["planned"]:
                p.tokens = [tokens.get(p.request.request_id, 0)]
        self.timeline.append({"active": len(self.scheduler.running), "waiting": len(self.scheduler.waiting),
                              "tokens": sum(len(p.tokens) for p in current["planned"])})
        return emitted

    def _launch(self, planned, behind=None) -> dict:
        """Queue a step and its sampling; ``behind``: the step whose sampled tokens are this step's
        input (every entry one token, same requests in the same order)."""
        entries = [StepEntry(p.request.request_id, p.tokens if behind is None else [0],
                             [len(p.tokens) - 1] if p.sample else []) for p in planned]
        ahead = 0 if behind is None else 1          # tokens the requests will have drawn before this step
        self.launch_log.append([(p.request.request_id, self.cache.length(p.request.request_id), len(p.tokens))
                                for p in planned])
        self.launches += 1
        if behind is not None:
            self.stats["queued_steps"] += 1
        device_tokens = self.sampler.device_tokens(behind["ticket"]) if behind is not None else None
        logits = self.runner.step(entries, device_tokens=device_tokens)
        ticket = None
        if logits is not None:
            self.runner.queue_status()
            rs = [p.request for p in planned if p.sample]
            ticket = self.sampler.launch(
                logits,
                [r.params.temperature for r in rs],
                [r.params.seed for r in rs],
                [len(r.generated) + ahead for r in rs],
            )
        return {"planned": planned, "ticket": ticket}

    def _following(self, current) -> list | None:
        """The step after ``current``, if it can be told before current's tokens are known: current
        holds one decode token of every live request, nobody waits to be admitted, and every request
        wants at least one more token after the one being drawn (an end-of-sequence token may still end
        one: see step()).  None: the next step is planned when the tokens are here."""
        planned = current["planned"]
        sched = self.scheduler
        if (not self.pipeline or current["ticket"] is None or sched.waiting or len(planned) != len(sched.running)
                or not self.runner.use_graphs):
            return None
        if not all(p.kind == "decode" and len(p.request.generated) + 1 < p.request.max_new_tokens for p in planned):
            return None
        return [Planned(p.request, [0], True, "decode") for p in planned]

    def _collect(self, step) -> list[int]:
        if step["ticket"] is None:
            return []
        sampled = self.sampler.collect(step["ticket"])
        self.runner.check_status(queued=True)    # the status word is sticky: a step without samples is
        return sampled                           # checked with the next one

    def run(self) -> dict:
        while not self.scheduler.idle or self._queued is not None:
            self.step()
        return {name: r.generated for name, r in self.scheduler.requests.items()}

    def cancel(self, request_id) -> None:
        self.scheduler.cancel(request_id)

    def snapshot(self) -> dict:
        return {"cache": self.cache.snapshot(), "scheduler": dict(self.scheduler.stats),
                "runner": dict(self.runner.stats), "engine": dict(self.stats)}
