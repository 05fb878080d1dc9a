"""The step function: one batch of (request, its next tokens) through the model, from the cache.

A step takes any mix of prompt portions and single decoded tokens, cut anywhere.  It runs only
the tokens it is given, as one batch, and returns float32 logits at the wanted places.  The
reference has no such function: it runs one whole prompt or one token of one request at a time
(mini_hisparse/model.py:160-226, mini_hisparse/engine.py:80-84).  The order inside a layer is
the reference's: project, rotate, append to the cache, then attend (model.py:169-170, 201).

Per step the host packs every index array the kernels need (token ids, positions, segment of
each token, block-table rows of the batch's requests, attention work items, wanted rows) into
one pinned buffer and sends it with a single copy.  A pure-decode batch can instead replay a
CUDA graph captured for its batch size; only the packed buffer changes between replays.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch

from ..cache.allocator import CapacityError
from ..cache.manager import CacheManager
from ..kernels import api as K
from ..kernels import build
from ..parts.base import CacheView, Segment, StepContext, StepPlanner, Workspace


@dataclass
class StepEntry:
    """One request's share of a step: its next tokens and the places whose logits are wanted."""

    request: object
    tokens: list[int]
    want: list[int] = field(default_factory=list)


class StepError(RuntimeError):
    pass


def _round_up(n: int, m: int) -> int:
    return -(-n // m) * m


class _Layout:
    """Offsets (in int32 words) of the packed per-step arrays for given sizes: the batch's own
    arrays, one block table per page group, and the arrays of every plan slot."""

    def __init__(self, T: int, S: int, R: int, widths: list[int], plan_caps: list[dict[str, int]]):
        self.T, self.S, self.R, self.widths, self.plan_caps = T, S, R, widths, plan_caps
        off = 0

        def take(n):
            nonlocal off
            start = off
            off += _round_up(max(n, 1), 4)   # keep every array 16-byte aligned
            return start

        self.tokens = take(T)
        self.positions = take(T)
        self.tok_seg = take(T)
        self.seg_slot = take(S)
        self.rows = take(R)
        self.tables = [take(S * w) for w in widths]
        self.plans = [{name: take(n) for name, n in caps.items()} for caps in plan_caps]
        self.total = off


class _Staging:
    """Two pinned host buffers used in turn, each guarded by an event of its last copy.  (Where no
    CUDA device is visible, as in tests of the packing alone, the buffers are plain host memory
    and there is nothing to guard.)"""

    def __init__(self):
        self.buffers = [None, None]
        self.events = [None, None]
        self.turn = 0
        self.cuda = torch.cuda.is_available()

    def next(self, words: int) -> tuple[torch.Tensor, int]:
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < words:
            buf = torch.empty(max(words, 1024) * 2, dtype=torch.int32)
            self.buffers[i] = buf.pin_memory() if self.cuda else buf
        return self.buffers[i], i

    def mark(self, i: int):
        if not self.cuda:
            return
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


@dataclass
class _PlanSlot:
    """One plan per step: the planner of the mixers of one page group whose plan keys are equal."""

    gid: int
    key: object
    planner: StepPlanner


class _DecodeGraph:
    """A captured step for exactly B single-token segments whose block tables are ``width`` wide, with
    what the planners hold constant in it (``fixed``, one value per plan slot)."""

    def __init__(self, runner: "ModelRunner", B: int, width: int, fixed: tuple):
        self.B = B
        self.ws = Workspace(runner.device)
        batch = runner.batch
        self.fixed = list(fixed)
        self.capturable = all(f is not None for f in self.fixed)
        caps = [slot.planner.capacity(B, B, f) for slot, f in zip(batch.slots, self.fixed)]
        self.layout = _Layout(B, B, B, [min(width, g.width) for g in runner.cache.page_groups], caps)
        self.meta = torch.zeros(self.layout.total, dtype=torch.int32, device=runner.device)
        self.facts = None       # the plans' host facts at capture: every replay must bring the same
        self.graph = None
        self.logits = None
        self.launches = 0


class BatchBuilder:
    """Turns a step's entries into the device arrays the kernels read.  It knows the cache manager
    and the planners that the cache's users bring, not the model: tests use it to run a single
    part.  What a planner's arrays mean is the planner's and its mixer's business."""

    def __init__(self, cache: CacheManager, device, sm_count: int | None = None):
        self.cache = cache
        self.device = torch.device(device)
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sm_count = sm_count
        self.meta = None
        self.staging = _Staging()
        self.slots: list[_PlanSlot] = []
        self.users: list[tuple[int | None, int | None]] = []     # user -> (cache entry, plan slot)

    def add_user(self, cache_entry: int | None, part=None) -> int:
        """Register a reader of cache entry ``cache_entry`` (a run entry's block or mixer; anything
        with plan_key() and planner()); returns the index that cache_view() takes."""
        slot = None
        where = self.cache.entry_group[cache_entry] if cache_entry is not None else None
        if where is not None and where[0] == "pages" and part is not None and part.plan_key() is not None:
            gid, key = where[1], part.plan_key()
            for i, sl in enumerate(self.slots):
                if sl.gid == gid and sl.key == key:
                    slot = i
                    break
            else:
                planner = part.planner(self.cache.cfg.page_size, self.sm_count)
                if planner is not None:
                    self.slots.append(_PlanSlot(gid, key, planner))
                    slot = len(self.slots) - 1
        self.users.append((cache_entry, slot))
        return len(self.users) - 1

    # ---- packing -----------------------------------------------------------------------------
    def segments(self, entries: list[StepEntry]) -> tuple[list[Segment], int]:
        segments, offset = [], 0
        seen = set()
        for e in entries:
            if e.request in seen:
                raise StepError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            n = len(e.tokens)
            if n < 1:
                raise StepError(f"request {e.request!r} brings no tokens")
            for w in e.want:
                if not 0 <= w < n:
                    raise StepError(f"request {e.request!r}: wanted place {w} is outside its {n} tokens")
            start = self.cache.length(e.request)
            segments.append(Segment(e.request, self.cache.slot(e.request), start, n, offset))
            offset += n
        return segments, offset

    @staticmethod
    def _put(buf: np.ndarray, offsets: dict[str, int], caps: dict[str, int], arrays: dict[str, np.ndarray],
             exact: bool = False) -> None:
        for name, cap in caps.items():
            arr = arrays[name]
            n = arr.size
            if n > cap or (exact and n != cap):
                raise StepError(f"plan array {name!r} has {n} words, the layout holds {cap}")
            region = buf[offsets[name]: offsets[name] + cap]
            region[:n] = arr.reshape(-1)
            region[n:] = 0

    def _fill(self, buf: np.ndarray, layout: _Layout, entries, segments):
        """Write the step's arrays into ``buf`` at the layout's offsets; return the wanted rows'
        count and the plans' host facts."""
        T = sum(s.count for s in segments)
        tokens = buf[layout.tokens : layout.tokens + T]
        positions = buf[layout.positions : layout.positions + T]
        tok_seg = buf[layout.tok_seg : layout.tok_seg + T]
        rows = []
        for si, (e, s) in enumerate(zip(entries, segments)):
            sl = slice(s.offset, s.offset + s.count)
            tokens[sl] = e.tokens
            positions[sl] = np.arange(s.start, s.start + s.count, dtype=np.int32)
            tok_seg[sl] = si
            buf[layout.seg_slot + si] = s.slot
            rows.extend(s.offset + w for w in e.want)
        if len(rows) > layout.R:
            raise StepError("more rows wanted than the layout holds")
        buf[layout.rows : layout.rows + len(rows)] = rows
        slots = [s.slot for s in segments]
        for gi, g in enumerate(self.cache.page_groups):
            table = self.cache.table_rows(g.gid, slots, layout.widths[gi])
            buf[layout.tables[gi] : layout.tables[gi] + table.size] = table.reshape(-1)
        facts = []
        for pi, slot in enumerate(self.slots):
            arrays, f = slot.planner.plan(segments, T)
            self._put(buf, layout.plans[pi], layout.plan_caps[pi], arrays)
            facts.append(f)
        return len(rows), facts

    def _fill_decode(self, buf: np.ndarray, layout: _Layout, entries, segments, fixed) -> list[dict]:
        """_fill for a batch of single decoded tokens that all want their logits, without loops
        over tokens: the arrays a captured decode graph reads.  Returns the plans' facts."""
        B = len(segments)
        starts = np.fromiter((s.start for s in segments), np.int64, B)
        slots = np.fromiter((s.slot for s in segments), np.intp, B)
        ar = np.arange(B, dtype=np.int32)
        buf[layout.tokens : layout.tokens + B] = [e.tokens[0] for e in entries]
        buf[layout.positions : layout.positions + B] = starts
        buf[layout.tok_seg : layout.tok_seg + B] = ar
        buf[layout.seg_slot : layout.seg_slot + B] = slots
        buf[layout.rows : layout.rows + B] = ar
        for gi, g in enumerate(self.cache.page_groups):
            width = layout.widths[gi]
            buf[layout.tables[gi] : layout.tables[gi] + B * width].reshape(B, width)[:] = g.table_np[slots, :width]
        facts = []
        for pi, slot in enumerate(self.slots):
            arrays, f = slot.planner.plan_decode(starts, fixed[pi])
            self._put(buf, layout.plans[pi], layout.plan_caps[pi], arrays, exact=True)
            facts.append(f)
        return facts

    def _views(self, meta: torch.Tensor, layout: _Layout, T: int, S: int, R: int, facts) -> dict:
        def v(off, n):
            return meta[off : off + n]

        plans = []
        for pi in range(len(self.slots)):
            d = {name: v(layout.plans[pi][name], cap) for name, cap in layout.plan_caps[pi].items()}
            d.update(facts[pi])
            plans.append(d)
        return {
            "tokens": v(layout.tokens, T),
            "positions": v(layout.positions, T),
            "tok_seg": v(layout.tok_seg, T),
            "seg_slot": v(layout.seg_slot, S),
            "rows": v(layout.rows, R) if R else None,
            "tables": [v(layout.tables[gi], S * w).view(S, w) for gi, w in enumerate(layout.widths)],
            "plans": plans,
        }

    def eager(self, entries, segments):
        """Pack and send the arrays of an eagerly launched step; returns the device views."""
        T = sum(s.count for s in segments)
        S = len(segments)
        R = sum(len(e.want) for e in entries)
        need_pages = max(1, max(-(-(s.start + s.count) // self.cache.cfg.page_size) for s in segments))
        widths = [min(need_pages, g.width) for g in self.cache.page_groups]
        caps = [slot.planner.capacity(T, S) for slot in self.slots]
        layout = _Layout(T, S, R, widths, caps)
        stage, turn = self.staging.next(layout.total)
        _, facts = self._fill(stage.numpy(), layout, entries, segments)
        if self.meta is None or self.meta.numel() < layout.total:
            self.meta = torch.empty(max(layout.total, 4096) * 2, dtype=torch.int32, device=self.device)
        self.meta[: layout.total].copy_(stage[: layout.total], non_blocking=True)
        self.staging.mark(turn)
        return self._views(self.meta, layout, T, S, R, facts)

    def context(self, rt, ws, status, views, segments) -> StepContext:
        return StepContext(
            rt=rt, ws=ws, T=sum(s.count for s in segments), segments=segments,
            tokens=views["tokens"], positions=views["positions"], tok_seg=views["tok_seg"],
            seg_slot=views["seg_slot"], status=status,
        )

    def cache_view(self, user: int, views: dict, writable: bool = True) -> CacheView | None:
        """The view of its cache entry for user ``user`` (see add_user) in one step."""
        entry, slot = self.users[user]
        where = self.cache.entry_group[entry] if entry is not None else None
        if where is None:
            return None
        kind, g, storage = self.cache.entry_storage(entry)
        if kind == "pages":
            meta = {"block_table": views["tables"][g.gid]}
            if slot is not None:
                meta.update(views["plans"][slot])
            return CacheView(g.need, g.gid, where[2], writable, storage,
                             page_size=self.cache.cfg.page_size, meta=meta)
        return CacheView(g.need, g.gid, where[2], writable, storage)


class ModelRunner:
    MAX_GRAPHS = 16      # captured decode graphs kept (each holds a workspace of its own); least recently used goes

    def __init__(self, model, cache: CacheManager, use_graphs: bool = True, sm_count: int | None = None,
                 graph_after: int = 1):
        self.model, self.cache = model, cache
        self.rt = model.rt
        self.device = self.rt.device
        for block in model.blocks:
            block.check_cache(cache.cfg.page_size)      # refuse now what a step would refuse half-way
        self.batch = BatchBuilder(cache, self.device, sm_count)
        for i, entry in enumerate(model.spec.order):
            self.batch.add_user(model.entry_cache[i], model.blocks[entry.layer])
        self.sm_count = self.batch.sm_count
        self.ws = Workspace(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        if hasattr(self.rt, "status"):
            self.rt.status = self.status
        self.use_graphs = use_graphs and model.graph_safe
        # A decode graph is captured at the ``graph_after``-th step that asks for it (a capture costs
        # several steps' time: a batch whose size changes every few steps is served faster without);
        # the steps before run launch by launch, with the same plans and kernels.
        self.graph_after = max(1, int(graph_after))
        self._asked: dict[tuple, int] = {}
        self.graphs: dict[tuple, _DecodeGraph] = {}
        self.observer = None
        self.side_stream = None
        self.side_events = None
        self.stats = {"steps": 0, "tokens": 0, "graph_steps": 0, "graph_captures": 0, "two_stream_layers": 0,
                      "prepared_steps": 0, "graph_deferred": 0}
        self._ahead = None      # index arrays of the next decode step, packed while the GPU ran this one
        build.build_all(model.kernel_modules())

    def _cache_views(self, views) -> list[CacheView | None]:
        return [self.batch.cache_view(i, views, writable=entry.cache_of is None)
                for i, entry in enumerate(self.model.spec.order)]

    # ---- the step -----------------------------------------------------------------------------
    @torch.inference_mode()
    def step(self, entries: list[StepEntry], device_tokens: torch.Tensor | None = None) -> torch.Tensor | None:
        """Run one batch.  Returns logits [wanted, vocab] float32 in the order of the entries and
        of their ``want`` lists, or None if nothing is wanted.  The tensor is scratch: it is
        overwritten by the next step.

        ``device_tokens`` (int32 on the device, one per entry, every entry a single token): the token
        ids are taken from there instead of from the entries, in stream order: a step can be queued
        behind the step that samples its input, before those tokens have reached the host."""
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        if device_tokens is not None:
            if any(len(e.tokens) != 1 for e in entries) or device_tokens.numel() != len(entries):
                raise StepError("tokens on the device stand for single-token entries, one each")
        for e in entries if device_tokens is None else ():
            if len(e.tokens) > 32:          # a prompt portion: one pass in numpy
                arr = np.asarray(e.tokens)
                bad = np.flatnonzero((arr < 0) | (arr >= vocab))
                if bad.size:
                    raise StepError(f"request {e.request!r}: token {int(arr[bad[0]])} is outside the vocabulary of {vocab}")
                continue
            for t in e.tokens:
                if not 0 <= t < vocab:
                    raise StepError(f"request {e.request!r}: token {t} is outside the vocabulary of {vocab}")
        segments, T = self.batch.segments(entries)
        maxpos = self.model.spec.max_positions
        for s in segments:
            if maxpos is not None and s.start + s.count > maxpos:
                raise StepError(
                    f"request {s.request!r} would reach position {s.start + s.count}, beyond "
                    f"max_position_embeddings {maxpos}"
                )
        for s in segments:
            self.cache.ensure(s.request, s.start + s.count)
        decode_only = all(s.count == 1 for s in segments) and all(e.want == [0] for e in entries)
        ahead, self._ahead = self._ahead, None       # what was packed ahead serves this step or none
        logits = None
        if self.use_graphs and decode_only and self.observer is None:   # a hook's calls are not replayed
            logits = self._step_graph(entries, segments, ahead, device_tokens)
        if logits is None:
            logits = self._step_eager(entries, segments, T, device_tokens)
        for s in segments:
            self.cache.advance(s.request, s.count)
        self.stats["steps"] += 1
        self.stats["tokens"] += T
        return logits

    def _step_eager(self, entries, segments, T, device_tokens=None):
        views = self.batch.eager(entries, segments)
        if device_tokens is not None:
            views["tokens"].copy_(device_tokens)
        return self._forward(self.ws, views, segments, T, side=True)

    def _forward(self, ws, views, segments, T, side: bool = False):
        ctx = self.batch.context(self.rt, ws, self.status, views, segments)
        if side:
            # a second stream for parts that have two independent kernels to run (attention over long
            # portions beside attention over decode tokens); never inside a graph capture
            if self.side_stream is None:
                self.side_stream = torch.cuda.Stream(self.device)
                self.side_events = (torch.cuda.Event(), torch.cuda.Event())
            ctx.extras["side_stream"] = self.side_stream
            ctx.extras["side_events"] = self.side_events
        caches = self._cache_views(views)
        with K.stream_scope():
            out = self.model.forward(ctx, caches, views["rows"], observer=self.observer)
        self.stats["two_stream_layers"] += ctx.extras.get("two_stream_layers", 0)
        return out

    def _graph_key(self, segments) -> tuple:
        """What a captured decode graph is made for: the batch size, the block-table width and what the
        planners want to hold constant for these histories."""
        B, width = len(segments), self._table_width(segments)
        starts = np.fromiter((s.start for s in segments), np.int64, B)
        max_keys = width * self.cache.cfg.page_size
        return B, width, tuple(slot.planner.decode_fixed_for(starts, max_keys) for slot in self.batch.slots)

    def _graph_for(self, key: tuple) -> _DecodeGraph:
        g = self.graphs.pop(key, None)
        if g is None:
            g = _DecodeGraph(self, *key)
            while len(self.graphs) >= self.MAX_GRAPHS:          # the dict keeps the order of last use
                old = self.graphs.pop(next(iter(self.graphs)))
                if self._ahead is not None and self._ahead["graph"] is old:
                    self._ahead = None
        self.graphs[key] = g
        return g

    def _step_graph(self, entries, segments, ahead=None, device_tokens=None):
        """The step through a captured graph, or None if a planner cannot hold its plan constant
        (then the step runs eagerly)."""
        B = len(segments)
        key = self._graph_key(segments)
        if key not in self.graphs and self.graph_after > 1:
            asked = self._asked.pop(key, 0) + 1
            if asked < self.graph_after:
                if len(self._asked) >= 256:
                    self._asked.pop(next(iter(self._asked)))
                self._asked[key] = asked
                self.stats["graph_deferred"] += 1
                return None
        g = self._graph_for(key)
        if not g.capturable:
            return None
        layout = g.layout
        if (ahead is not None and ahead["graph"] is g and g.graph is not None
                and ahead["who"] == [(s.request, s.slot, s.start) for s in segments]):
            # everything but the token ids was packed while the GPU ran the step before this one
            stage, turn = ahead["stage"], ahead["turn"]
            stage.numpy()[layout.tokens : layout.tokens + B] = [e.tokens[0] for e in entries]
            self.stats["prepared_steps"] += 1
        else:
            stage, turn = self.batch.staging.next(layout.total)
            facts = self.batch._fill_decode(stage.numpy(), layout, entries, segments, g.fixed)
            if g.facts is None:
                g.facts = facts
            elif facts != g.facts:
                raise StepError(f"a decode plan changed after its graph was captured: {facts} vs {g.facts}")
        g.meta.copy_(stage[: layout.total], non_blocking=True)
        self.batch.staging.mark(turn)
        if device_tokens is not None:
            g.meta[layout.tokens : layout.tokens + B].copy_(device_tokens)
        if g.graph is None:
            views = self.batch._views(g.meta, layout, B, B, B, g.facts)
            # one eager run sizes the workspace and warms the kernels up, then the capture
            g.logits = self._forward(g.ws, views, segments, B)
            g.ws.frozen = True
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            before = K.launches
            with torch.cuda.graph(graph):
                g.logits = self._forward(g.ws, views, segments, B)
            g.launches = K.launches - before
            K.launches = before + 0          # the capture launched nothing
            g.graph = graph
            # the capture itself ran nothing: the eager run above already produced this step
            self.stats["graph_steps"] += 1
            self.stats["graph_captures"] += 1
            return g.logits
        g.graph.replay()
        K.launches += g.launches
        self.stats["graph_steps"] += 1
        return g.logits

    def prepare_decode_ahead(self, requests: list, take_pages: bool = True) -> None:
        """Pack the index arrays of the NEXT step, assuming that it decodes one token for each of
        ``requests`` (in this order) and for nobody else.  Called between a decode step's launch and
        the wait for its result: the host would idle meanwhile, and positions, block tables and the
        plans of the next step do not depend on the tokens still being computed.  If the next step
        turns out differently (a request finished, another arrived), what was packed is dropped and
        the step is packed as usual.  Pages the next positions need are taken now (a request that
        ends after all gives them back with its others); with ``take_pages`` False nothing is
        packed when a page would have to be taken (for callers whose pool has no page to spare)."""
        self._ahead = None
        if not self.use_graphs or not requests:
            return
        maxpos = self.model.spec.max_positions
        entries = [StepEntry(r, [0], [0]) for r in requests]
        for e in entries:
            length = self.cache.length(e.request)
            if maxpos is not None and length + 1 > maxpos:
                return
            if not take_pages:
                if not self.cache.has_pages(e.request, length + 1):
                    return
                continue
            try:
                self.cache.ensure(e.request, length + 1)
            except CapacityError:
                return          # the step itself will say so, if it comes to that
        segments, _ = self.batch.segments(entries)
        g = self.graphs.get(self._graph_key(segments))
        if g is None or g.graph is None:
            return              # that step will capture its graph: nothing to gain
        stage, turn = self.batch.staging.next(g.layout.total)
        if self.batch._fill_decode(stage.numpy(), g.layout, entries, segments, g.fixed) != g.facts:
            return
        self._ahead = {"graph": g, "stage": stage, "turn": turn,
                       "who": [(s.request, s.slot, s.start) for s in segments]}

    def _table_width(self, segments) -> int:
        """Block-table width of a decode graph: a power of two, so a graph is re-captured only when
        contexts double."""
        pages = max(-(-(s.start + 1) // self.cache.cfg.page_size) for s in segments)
        width = 16
        while width < pages:
            width *= 2
        return width

    # ---- the status word ------------------------------------------------------------------------
    STATUS_BITS = {
        1: "a token id outside the vocabulary reached the embedding",
        2: "a position had no valid page in its block table",
        4: "a bounded wait in the tensor-core matrix product ran out",
        8: "a bounded wait in the TMA-fed attention kernel ran out",
        16: "a bounded wait in the tcgen05 attention kernel ran out",
        32: "a token's keys were split into more parts than the attention kernel merges",
    }

    @classmethod
    def status_message(cls, bits: int) -> str:
        what = [text for bit, text in cls.STATUS_BITS.items() if bits & bit]
        rest = bits & ~sum(cls.STATUS_BITS)
        if rest:
            what.append(f"unknown status bits {rest:#x}")
        return "; ".join(what)

    def queue_status(self) -> None:
        """Start the copy of the status word to the host; read it with check_status(queued=True)
        after the stream has been synchronised (saves a synchronisation of its own)."""
        self.status_host.copy_(self.status, non_blocking=True)

    def check_status(self, queued: bool = False) -> None:
        """Raise StepError if a kernel flagged a fault (ids outside the table, pages outside the pool,
        a bounded wait that ran out).  Before raising, everything that such a kernel may have left
        behind is put back: the status word, and the counters and flags that kernels hand to their
        next launch as zero (see reset_after_error)."""
        bits = int(self.status_host.item()) if queued else int(self.status.item())
        if bits:
            self.reset_after_error()
            raise StepError(self.status_message(bits))

    def reset_after_error(self) -> None:
        """A kernel that gave up may have left its self-resetting scratch non-zero: the counters of
        the key-split merge in every workspace (this runner's and each captured graph's) and the
        flags of the persistent product.  Zero them and the status word, so that the next step
        starts clean; what was packed ahead is dropped."""
        torch.cuda.synchronize(self.device)
        self.status.zero_()
        for ws in [self.ws] + [g.ws for g in self.graphs.values()]:
            ws.zero_self_resetting()
        scratch = getattr(self.rt, "_scratch", None)
        if scratch is not None:
            scratch[1].zero_()
        self._ahead = None
