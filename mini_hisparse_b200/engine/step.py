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
from ..parts.attention import ITEM_INTS, ROW_TILE, plan_attention, plan_capacity, plan_decode
from ..parts.base import CacheView, Segment, StepContext, Workspace
from ..parts.spec import PagedKVNeed


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
    """Offsets (in int32 words) of the packed per-step arrays for given sizes."""

    def __init__(self, T: int, S: int, R: int, groups: list[tuple[int, int]]):
        self.T, self.S, self.R, self.groups = T, S, R, groups
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
        self.group_offsets = []
        for items, width in groups:
            self.group_offsets.append(
                {
                    "block_table": take(S * width),
                    "items": take(items * ITEM_INTS),
                    "tok_part_row": take(T),
                    "tok_nsplit": take(T),
                }
            )
        self.total = off


class _Staging:
    """Two pinned host buffers used in turn, each guarded by an event of its last copy."""

    def __init__(self):
        self.buffers = [None, None]
        self.events = [None, None]
        self.turn = 0

    def next(self, words: int) -> tuple[torch.Tensor, int]:
        i = self.turn
        self.turn ^= 1
        if self.events[i] is not None:
            self.events[i].synchronize()
        buf = self.buffers[i]
        if buf is None or buf.numel() < words:
            buf = torch.empty(max(words, 1024) * 2, dtype=torch.int32).pin_memory()
            self.buffers[i] = buf
        return buf, i

    def mark(self, i: int):
        ev = self.events[i] or torch.cuda.Event()
        ev.record()
        self.events[i] = ev


class _DecodeGraph:
    """A captured step for exactly B single-token segments whose block tables are ``width`` wide."""

    def __init__(self, runner: "ModelRunner", B: int, width: int):
        self.B = B
        self.ws = Workspace(runner.device)
        max_keys = width * runner.cache.cfg.page_size
        self.nsplit = [runner.batch.decode_splits(g.need, B, max_keys) for g in runner.cache.page_groups]
        caps = []
        for g, ns in zip(runner.cache.page_groups, self.nsplit):
            groups = g.need.q_heads // g.need.kv_heads
            chunks = 1 if groups <= ROW_TILE else -(-groups // ROW_TILE)
            caps.append((B * ns * chunks, min(width, g.width)))
        self.layout = _Layout(B, B, B, caps)
        self.meta = torch.zeros(self.layout.total, dtype=torch.int32, device=runner.device)
        self.graph = None
        self.logits = None
        self.launches = 0


class BatchBuilder:
    """Turns a step's entries into the device arrays the kernels read.  It knows the cache
    manager, not the model: tests use it to run a single part."""

    def __init__(self, cache: CacheManager, device, sm_count: int | None = None):
        self.cache = cache
        self.device = torch.device(device)
        if sm_count is None:
            sm_count = torch.cuda.get_device_properties(self.device).multi_processor_count
        self.sm_count = sm_count
        self.meta = None
        self.staging = _Staging()

    # ---- planning ----------------------------------------------------------------------------
    def decode_splits(self, need: PagedKVNeed, B: int, max_keys: int) -> int:
        """Key splits per decoded token for a batch of B with at most ``max_keys`` cached keys: as
        many CTAs as are resident at once (two per SM), never more, so that no CTA waits for a
        second wave, and no split shorter than MIN_KEYS_PER_SPLIT keys."""
        from ..parts.attention import MAX_SPLITS, MIN_KEYS_PER_SPLIT, ROW_TILE

        groups = need.q_heads // need.kv_heads
        chunks = 1 if groups <= ROW_TILE else -(-groups // ROW_TILE)
        ctas = B * need.kv_heads * chunks
        return max(1, min(MAX_SPLITS, (2 * self.sm_count) // ctas, max_keys // MIN_KEYS_PER_SPLIT))

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

    def _fill(self, buf: np.ndarray, layout: _Layout, entries, segments, fixed_nsplit=None):
        """Write the step's arrays into ``buf`` at the layout's offsets; return per-group facts."""
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
        facts = []
        for gi, g in enumerate(self.cache.page_groups):
            offs = layout.group_offsets[gi]
            cap_items, width = layout.groups[gi]
            table = self.cache.table_rows(g.gid, [s.slot for s in segments], width)
            buf[offs["block_table"] : offs["block_table"] + table.size] = table.reshape(-1)
            plan = plan_attention(g.need, segments, T, self.sm_count,
                                  fixed_nsplit=None if fixed_nsplit is None else fixed_nsplit[gi])
            n_items = plan.items.shape[0]
            if n_items > cap_items:
                raise StepError(f"attention plan has {n_items} items, layout holds {cap_items}")
            region = buf[offs["items"] : offs["items"] + cap_items * ITEM_INTS]
            region[: n_items * ITEM_INTS] = plan.items.reshape(-1)
            region[n_items * ITEM_INTS :] = 0
            buf[offs["tok_part_row"] : offs["tok_part_row"] + T] = plan.tok_part_row
            buf[offs["tok_nsplit"] : offs["tok_nsplit"] + T] = plan.tok_nsplit
            facts.append({"n_small": plan.n_small, "n_big": plan.n_big, "part_rows": plan.part_rows,
                          "any_split": bool(plan.part_rows), "big_split": plan.big_split})
        return len(rows), facts

    def _fill_decode(self, buf: np.ndarray, layout: _Layout, entries, segments, nsplit):
        """_fill for a batch of single decoded tokens that all want their logits, without loops
        over tokens: the arrays a captured decode graph reads."""
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
            offs = layout.group_offsets[gi]
            cap_items, width = layout.groups[gi]
            buf[offs["block_table"] : offs["block_table"] + B * width].reshape(B, width)[:] = g.table_np[slots, :width]
            plan = plan_decode(g.need, starts, nsplit[gi])
            n = plan.items.shape[0]
            if n != cap_items:
                raise StepError(f"decode plan has {n} items, the graph was captured for {cap_items}")
            buf[offs["items"] : offs["items"] + n * ITEM_INTS] = plan.items.reshape(-1)
            buf[offs["tok_part_row"] : offs["tok_part_row"] + B] = plan.tok_part_row
            buf[offs["tok_nsplit"] : offs["tok_nsplit"] + B] = plan.tok_nsplit

    def _views(self, meta: torch.Tensor, layout: _Layout, T: int, S: int, R: int, facts, launch_items=None):
        def v(off, n):
            return meta[off : off + n]

        group_meta = []
        for gi, g in enumerate(self.cache.page_groups):
            offs = layout.group_offsets[gi]
            cap_items, width = layout.groups[gi]
            f = facts[gi]
            group_meta.append(
                {
                    "block_table": v(offs["block_table"], S * width).view(S, width),
                    "items": v(offs["items"], cap_items * ITEM_INTS),
                    "n_small": cap_items if launch_items else f["n_small"],
                    "n_big": 0 if launch_items else f["n_big"],
                    "tok_part_row": v(offs["tok_part_row"], T),
                    "tok_nsplit": v(offs["tok_nsplit"], T),
                    "part_rows_cap": f["part_rows"],
                    "any_split": f["any_split"],
                    "big_split": f.get("big_split", False),
                }
            )
        return {
            "tokens": v(layout.tokens, T),
            "positions": v(layout.positions, T),
            "tok_seg": v(layout.tok_seg, T),
            "seg_slot": v(layout.seg_slot, S),
            "rows": v(layout.rows, R) if R else None,
            "groups": group_meta,
        }

    def eager(self, entries, segments):
        """Pack and send the arrays of an eagerly launched step; returns the device views."""
        T = sum(s.count for s in segments)
        S = len(segments)
        R = sum(len(e.want) for e in entries)
        caps = []
        for g in self.cache.page_groups:
            items, _ = plan_capacity(g.need, T, S)
            width = max(1, max(-(-(s.start + s.count) // self.cache.cfg.page_size) for s in segments))
            caps.append((items, min(width, g.width)))
        layout = _Layout(T, S, R, caps)
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

    def cache_view(self, entry: int, group_meta, writable: bool = True) -> CacheView | None:
        """The view of cache entry ``entry`` for one step."""
        where = self.cache.entry_group[entry]
        if where is None:
            return None
        kind, g, storage = self.cache.entry_storage(entry)
        if kind == "pages":
            return CacheView(g.need, g.gid, where[2], writable, storage,
                             page_size=self.cache.cfg.page_size, meta=group_meta[g.gid])
        return CacheView(g.need, g.gid, where[2], writable, storage)


class ModelRunner:
    def __init__(self, model, cache: CacheManager, use_graphs: bool = True, sm_count: int | None = None):
        self.model, self.cache = model, cache
        self.rt = model.rt
        self.device = self.rt.device
        self.batch = BatchBuilder(cache, self.device, sm_count)
        self.sm_count = self.batch.sm_count
        self.ws = Workspace(self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        self.status_host = torch.zeros(1, dtype=torch.int32).pin_memory()
        if hasattr(self.rt, "status"):
            self.rt.status = self.status
        self.use_graphs = use_graphs and model.graph_safe
        self.graphs: dict[tuple[int, int], _DecodeGraph] = {}
        self.observer = None
        self.side_stream = None
        self.side_events = None
        self.stats = {"steps": 0, "tokens": 0, "graph_steps": 0, "two_stream_layers": 0, "prepared_steps": 0}
        self._ahead = None      # index arrays of the next decode step, packed while the GPU ran this one
        build.build_all(model.kernel_modules())

    def _cache_views(self, group_meta) -> list[CacheView | None]:
        return [
            self.batch.cache_view(self.model.entry_cache[i], group_meta, writable=entry.cache_of is None)
            for i, entry in enumerate(self.model.spec.order)
        ]

    # ---- the step -----------------------------------------------------------------------------
    @torch.inference_mode()
    def step(self, entries: list[StepEntry]) -> torch.Tensor | None:
        """Run one batch.  Returns logits [wanted, vocab] float32 in the order of the entries and
        of their ``want`` lists, or None if nothing is wanted.  The tensor is scratch: it is
        overwritten by the next step."""
        if not entries:
            return None
        vocab = self.model.spec.vocab_size
        for e in entries:
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
        if self.use_graphs and decode_only:
            logits = self._step_graph(entries, segments, ahead)
        else:
            logits = self._step_eager(entries, segments, T)
        for s in segments:
            self.cache.advance(s.request, s.count)
        self.stats["steps"] += 1
        self.stats["tokens"] += T
        return logits

    def _step_eager(self, entries, segments, T):
        views = self.batch.eager(entries, segments)
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
        caches = self._cache_views(views["groups"])
        with K.stream_scope():
            out = self.model.forward(ctx, caches, views["rows"], observer=self.observer)
        self.stats["two_stream_layers"] += ctx.extras.get("two_stream_layers", 0)
        return out

    def _step_graph(self, entries, segments, ahead=None):
        B = len(segments)
        width = self._table_width(segments)
        g = self.graphs.get((B, width))
        if g is None:
            g = self.graphs[(B, width)] = _DecodeGraph(self, B, width)
        layout = g.layout
        if (ahead is not None and ahead["graph"] is g and g.graph is not None
                and ahead["who"] == [(s.request, s.slot, s.start) for s in segments]):
            # everything but the token ids was packed while the GPU ran the step before this one
            stage, turn = ahead["stage"], ahead["turn"]
            stage.numpy()[layout.tokens : layout.tokens + B] = [e.tokens[0] for e in entries]
            self.stats["prepared_steps"] += 1
        else:
            stage, turn = self.batch.staging.next(layout.total)
            self.batch._fill_decode(stage.numpy(), layout, entries, segments, g.nsplit)
        g.meta.copy_(stage[: layout.total], non_blocking=True)
        self.batch.staging.mark(turn)
        if g.graph is None:
            # fixed facts for the capture: every item slot is launched, splits are constant
            fixed = []
            for gi, pg in enumerate(self.cache.page_groups):
                fixed.append({"n_small": layout.groups[gi][0], "n_big": 0, "part_rows": B * g.nsplit[gi],
                              "any_split": g.nsplit[gi] > 1})
            views = self.batch._views(g.meta, layout, B, B, B, fixed, launch_items=True)
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
            return g.logits
        g.graph.replay()
        K.launches += g.launches
        self.stats["graph_steps"] += 1
        return g.logits

    def prepare_decode_ahead(self, requests: list) -> None:
        """Pack the index arrays of the NEXT step, assuming that it decodes one token for each of
        ``requests`` (in this order) and for nobody else.  Called between a decode step's launch and
        the wait for its result: the host would idle meanwhile, and positions, block tables and the
        attention plan of the next step do not depend on the tokens still being computed.  If the
        next step turns out differently (a request finished, another arrived), what was packed is
        dropped and the step is packed as usual.  Pages the next positions need are taken now: a
        request that ends after all gives them back with its others."""
        self._ahead = None
        if not self.use_graphs or not requests:
            return
        maxpos = self.model.spec.max_positions
        entries = [StepEntry(r, [0], [0]) for r in requests]
        for e in entries:
            length = self.cache.length(e.request)
            if maxpos is not None and length + 1 > maxpos:
                return
            try:
                self.cache.ensure(e.request, length + 1)
            except CapacityError:
                return          # the step itself will say so, if it comes to that
        segments, _ = self.batch.segments(entries)
        g = self.graphs.get((len(segments), self._table_width(segments)))
        if g is None or g.graph is None:
            return              # that step will capture its graph: nothing to gain
        stage, turn = self.batch.staging.next(g.layout.total)
        self.batch._fill_decode(stage.numpy(), g.layout, entries, segments, g.nsplit)
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

    def queue_status(self) -> None:
        """Start the copy of the status word to the host; read it with check_status(queued=True)
        after the stream has been synchronised (saves a synchronisation of its own)."""
        self.status_host.copy_(self.status, non_blocking=True)

    def check_status(self, queued: bool = False) -> None:
        """Raise if a kernel flagged a bad index (ids outside the table, pages outside the pool)."""
        bits = int(self.status_host.item()) if queued else int(self.status.item())
        if bits:
            self.status.zero_()
            what = []
            if bits & 1:
                what.append("a token id outside the vocabulary reached the embedding")
            if bits & 2:
                what.append("a position had no valid page in its block table")
            if bits & 4:
                what.append("a bounded wait in the tensor-core matrix product ran out")
            if bits & 8:
                what.append("a bounded wait in the TMA-fed attention kernel ran out")
            if bits & 16:
                what.append("a bounded wait in the tcgen05 attention kernel ran out")
            if bits & 32:
                what.append("a token's keys were split into more parts than the attention kernel merges")
            raise StepError("; ".join(what) or f"kernel status {bits}")
