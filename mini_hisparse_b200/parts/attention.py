"""Grouped-query attention over the paged cache, and the plan of its work for one step."""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np
import torch

from ..kernels import api as K
from .base import CacheView, Mixer, Product, StepContext, StepPlanner
from .registry import POSITIONS, register_mixer
from .spec import PagedKVNeed, ParamSpec, PartSpec

ROW_TILE = 16          # query rows (tokens x heads of one group) per CTA of the attention kernel
KEY_TILE = 64          # split boundaries are multiples of the kernels' key tile
ITEM_INTS = 8
MIN_KEYS_PER_SPLIT = 256
SPLIT_MAX_TOKENS = 16  # only short segments (decode tokens, tiny portions) are split along the keys
MAX_SPLITS = 64
MAX_BIG_SPLITS = 8       # key splits of a long portion's tile (tcgen05 kernel only)
BIG_SPLIT_ITEMS = 1024   # long-portion tiles are only split while their items stay below this
BIG_SPLIT_ROWS = 4096    # ... and their partial rows (tokens x splits) below this
MIN_KEYS_PER_BIG_SPLIT = 512


@dataclass(frozen=True)
class AttentionShape:
    """What the plan of a step's attention depends on: head counts, the window, and the query rows
    per tile that the kernel for long portions takes (a kernel's choice, made by the mixer)."""

    q_heads: int
    kv_heads: int
    window: int | None = None
    tile_rows: int = ROW_TILE


@dataclass
class AttentionPlan:
    """Host arrays of one page group for one step (see csrc/attention_simt.cu for the item layout).
    Items of short segments (tiles of at most ROW_TILE rows, possibly split along the keys) come
    first, then the items of long portions (tiles of at most ``need.tile_rows`` rows)."""

    items: np.ndarray          # [n_small + n_big, 8] int32
    n_small: int
    n_big: int
    tok_part_row: np.ndarray   # [T] int32
    tok_nsplit: np.ndarray     # [T] int32: 0 = written directly
    part_rows: int
    big_split: bool = False    # some long-portion tiles are split along the keys (merged by attention_combine)


def _tiling(groups: int, rows: int):
    """Head chunks and tokens per tile for tiles of ``rows`` query rows."""
    if groups <= rows:
        return [(0, groups)], rows // groups
    return [(h, min(rows, groups - h)) for h in range(0, groups, rows)], 1


def plan_attention(need: AttentionShape, segments, T: int, sm_count: int = 148,
                   fixed_nsplit: int | None = None) -> AttentionPlan:
    """Cut the step's attention into items.

    A tile is a run of tokens of one segment times the heads of one KV group (or a chunk of
    them, if a group has more heads than a tile has rows).  Its keys are [kv_begin, kv_end):
    everything up to its last token, minus what a window has passed.  Short segments (decode
    tokens, tiny portions) get tiles of ROW_TILE rows and, when their histories are long, are
    split along the keys so that a small batch still fills the GPU; with ``fixed_nsplit`` every
    short segment gets exactly that many splits (a captured graph needs a fixed launch size),
    empty ones included.  Long portions get tiles of ``need.tile_rows`` rows; when there are fewer
    of them than SMs (a portion of some dozens of tokens far into a long prompt) and the tiles are
    the tcgen05 kernel's, they are split along the keys too, into the number of parts that fills
    a round of CTAs best.
    """
    groups = need.q_heads // need.kv_heads
    window = need.window or 0
    small_chunks, small_tpt = _tiling(groups, ROW_TILE)
    big_chunks, big_tpt = _tiling(groups, need.tile_rows)
    small_tiles, big_items = [], []
    for si, seg in enumerate(segments):
        short = seg.count <= SPLIT_MAX_TOKENS
        tpt = small_tpt if short else big_tpt
        for a in range(0, seg.count, tpt):
            nt = min(tpt, seg.count - a)
            first_pos = seg.start + a
            kv_end = first_pos + nt
            kv_begin = max(0, first_pos - window + 1) if window else 0
            if short:
                small_tiles.append((si, seg.offset + a, nt, kv_begin, kv_end))
            else:
                for h0, nh in big_chunks:
                    big_items.append((si, seg.offset + a, nt, h0, nh, kv_begin, kv_end, -1))
    # keys a CTA of a short segment should walk: an even share of all their keys over two CTAs per
    # SM, so that a long history beside short ones is cut into more parts and no CTA runs alone at
    # the end
    small_keys = sum(t[4] - t[3] for t in small_tiles) * len(small_chunks) * need.kv_heads
    target = max(MIN_KEYS_PER_SPLIT, -(-small_keys // (2 * sm_count)))
    target = -(-target // KEY_TILE) * KEY_TILE
    items = []
    tok_part_row = np.zeros(T, np.int32)
    tok_nsplit = np.zeros(T, np.int32)
    part_rows = 0
    for si, tok0, nt, kv_begin, kv_end in small_tiles:
        nsplit = 1
        if fixed_nsplit is not None:
            nsplit = fixed_nsplit
        else:
            fit = max(1, (kv_end - kv_begin) // MIN_KEYS_PER_SPLIT)
            nsplit = max(1, min(-(-(kv_end - kv_begin) // target), fit, MAX_SPLITS))
        if nsplit == 1:
            for h0, nh in small_chunks:
                items.append((si, tok0, nt, h0, nh, kv_begin, kv_end, -1))
            continue
        span = kv_end - kv_begin
        chunk = -(-span // nsplit)
        chunk = -(-chunk // KEY_TILE) * KEY_TILE
        for t in range(tok0, tok0 + nt):
            tok_part_row[t] = part_rows
            tok_nsplit[t] = nsplit
            part_rows += nsplit
        for sp in range(nsplit):
            b = min(kv_end, kv_begin + sp * chunk)
            e = min(kv_end, b + chunk)
            for h0, nh in small_chunks:
                items.append((si, tok0, nt, h0, nh, b, e, sp))
    n_small = len(items)
    big_split = False
    # A CTA alone on its SM walks its key tiles nearly twice as fast as one that shares the SM, so
    # splitting only pays while there are fewer CTAs than SMs (measured: 160 CTAs of 50 tiles took
    # 49 us, the same work as 480 CTAs 56 us plus the merge).
    slots = sm_count
    n_big_ctas = len(big_items) * need.kv_heads
    if big_items and need.tile_rows == 128 and fixed_nsplit is None and n_big_ctas < slots:
        tiles = [-(-(it[6] - it[5]) // KEY_TILE) for it in big_items]
        avg = sum(tiles) / len(tiles)
        big_tokens = sum(it[2] for it in big_items) // len(big_chunks)
        fixed = 3.0                            # a CTA's start and end, in key tiles
        best, best_cost = 1, -(-n_big_ctas // slots) * (avg + fixed)
        for sp in range(2, MAX_BIG_SPLITS + 1):
            if (avg * KEY_TILE / sp < MIN_KEYS_PER_BIG_SPLIT or len(big_items) * sp > BIG_SPLIT_ITEMS
                    or big_tokens * sp > BIG_SPLIT_ROWS):
                break
            cost = -(-n_big_ctas * sp // slots) * (avg / sp + fixed)
            if cost < 0.9 * best_cost:
                best, best_cost = sp, cost
        if best > 1:
            cut, seen = [], set()
            for it in big_items:
                si, tok0, nt, h0, nh, kv_begin, kv_end, _ = it
                span = kv_end - kv_begin
                if span < best * MIN_KEYS_PER_BIG_SPLIT // 2:
                    cut.append(it)
                    continue
                if (si, tok0) not in seen:      # the head chunks of a tile share its partial rows
                    seen.add((si, tok0))
                    for t in range(tok0, tok0 + nt):
                        tok_part_row[t] = part_rows
                        tok_nsplit[t] = best
                        part_rows += best
                chunk = -(-(-(-span // best)) // KEY_TILE) * KEY_TILE
                for sp in range(best):
                    b = min(kv_end, kv_begin + sp * chunk)
                    cut.append((si, tok0, nt, h0, nh, b, min(kv_end, b + chunk), sp))
            big_items, big_split = cut, True
    # long tiles first: the CTAs that walk the most keys must not be the last to start
    big_items.sort(key=lambda it: it[5] - it[6])
    arr = np.asarray(items + big_items, np.int32).reshape(-1, ITEM_INTS)
    return AttentionPlan(arr, n_small, len(big_items), tok_part_row, tok_nsplit, part_rows, big_split)


def plan_decode(need: AttentionShape, starts: np.ndarray, nsplit: int) -> AttentionPlan:
    """The plan of a batch of single decoded tokens (token i belongs to segment i and sits at
    position starts[i]) with exactly ``nsplit`` key splits each: what plan_attention gives for such
    a batch with fixed_nsplit, computed with arrays instead of loops."""
    B = len(starts)
    groups = need.q_heads // need.kv_heads
    chunks, _ = _tiling(groups, ROW_TILE)
    C = len(chunks)
    kv_end = starts.astype(np.int64) + 1
    kv_begin = np.maximum(0, starts - need.window + 1) if need.window else np.zeros(B, np.int64)
    items = np.empty((B, nsplit, C, ITEM_INTS), np.int32)
    seg = np.arange(B, dtype=np.int32)
    items[..., 0] = seg[:, None, None]
    items[..., 1] = seg[:, None, None]
    items[..., 2] = 1
    items[..., 3] = np.asarray([h for h, _ in chunks], np.int32)[None, None, :]
    items[..., 4] = np.asarray([n for _, n in chunks], np.int32)[None, None, :]
    if nsplit == 1:
        items[..., 5] = kv_begin[:, None, None]
        items[..., 6] = kv_end[:, None, None]
        items[..., 7] = -1
        return AttentionPlan(items.reshape(-1, ITEM_INTS), B * C, 0, np.zeros(B, np.int32),
                             np.zeros(B, np.int32), 0)
    span = kv_end - kv_begin
    chunk = -(-(-(-span // nsplit)) // KEY_TILE) * KEY_TILE
    ks = np.arange(nsplit, dtype=np.int64)
    b = np.minimum(kv_end[:, None], kv_begin[:, None] + ks[None, :] * chunk[:, None])
    e = np.minimum(kv_end[:, None], b + chunk[:, None])
    items[..., 5] = b[:, :, None]
    items[..., 6] = e[:, :, None]
    items[..., 7] = ks[None, :, None]
    return AttentionPlan(items.reshape(-1, ITEM_INTS), B * nsplit * C, 0,
                         (seg * nsplit).astype(np.int32), np.full(B, nsplit, np.int32), B * nsplit)


def plan_capacity(need: AttentionShape, max_tokens: int, max_segments: int,
                  fixed_nsplit: int | None = None) -> tuple[int, int]:
    """Upper bounds (items, partial rows) for a step of at most max_tokens / max_segments."""
    groups = need.q_heads // need.kv_heads
    small_chunks, small_tpt = _tiling(groups, ROW_TILE)
    big_chunks, big_tpt = _tiling(groups, need.tile_rows)
    splits = fixed_nsplit or MAX_SPLITS
    # every segment may end with a ragged tile; only short segments are split
    big = (max_tokens // big_tpt + max_segments) * len(big_chunks) + BIG_SPLIT_ITEMS
    short_tokens = min(max_tokens, max_segments * SPLIT_MAX_TOKENS)
    small = (short_tokens // small_tpt + max_segments) * len(small_chunks) * splits
    return big + small, short_tokens * splits + BIG_SPLIT_ROWS


class AttentionPlanner(StepPlanner):
    """The plan of grouped-query attention for the step function: work items, and for every token
    the first of its partial rows and the number of its key splits."""

    def __init__(self, shape: AttentionShape, sm_count: int, clusters_of=None, max_cluster: int = 0):
        """``clusters_of(n)``: how many clusters of n CTAs the mixer's decode kernel can run at once, if
        it merges a token's key splits inside a cluster of up to ``max_cluster`` CTAs (None: it does not)."""
        self.shape, self.sm_count = shape, sm_count
        self.clusters_of, self.max_cluster = clusters_of, max_cluster
        self._uneven = {}        # decode_fixed_for's answers
        groups = shape.q_heads // shape.kv_heads
        self.chunks = 1 if groups <= ROW_TILE else -(-groups // ROW_TILE)

    def capacity(self, max_tokens, max_segments, fixed=None):
        if fixed is not None:            # a captured graph of single tokens: exactly these many
            return {"items": max_segments * fixed[0] * fixed[1] * self.chunks * ITEM_INTS, "tok_part_row": max_tokens,
                    "tok_nsplit": max_tokens}
        items, _ = plan_capacity(self.shape, max_tokens, max_segments)
        return {"items": items * ITEM_INTS, "tok_part_row": max_tokens, "tok_nsplit": max_tokens}

    @staticmethod
    def _out(plan: AttentionPlan, decode_nsplit: int = 0, decode_groups: int = 1):
        arrays = {"items": plan.items.reshape(-1), "tok_part_row": plan.tok_part_row, "tok_nsplit": plan.tok_nsplit}
        # decode_nsplit > 0: the step is single tokens only (token i = segment i), every one with
        # decode_groups x decode_nsplit equal shares of keys, decode_nsplit of them to a cluster: what a
        # kernel that plans for itself needs to know
        facts = {"n_small": plan.n_small, "n_big": plan.n_big, "part_rows_cap": plan.part_rows,
                 "any_split": bool(plan.part_rows), "big_split": plan.big_split, "decode_nsplit": decode_nsplit,
                 "decode_groups": decode_groups}
        return arrays, facts

    def plan(self, segments, T, fixed=None):
        if fixed is None and T == len(segments) and all(s.offset == i for i, s in enumerate(segments)):
            # single tokens only: the plan of a captured decode graph, so that a step does not
            # depend on whether it is replayed or launched
            starts = np.fromiter((s.start for s in segments), np.int64, T)
            return self.plan_decode(starts, self.decode_fixed_for(starts, int(starts.max()) + 1))
        every = None if fixed is None else fixed[0] * fixed[1]
        return self._out(plan_attention(self.shape, segments, T, self.sm_count, fixed_nsplit=every))

    # what a CTA costs beside its keys (the query and the merge) and what a launch of attention_combine
    # costs the step, in key tiles of streaming time
    CTA_FIXED_TILES = 3.5
    COMBINE_TILES = 8.0
    STREAMS = 240.0          # CTAs streaming at a lone CTA's rate that the memory can feed

    def decode_fixed(self, segments_count, max_positions):
        """Key shares per decoded token for a batch of B with at most ``max_positions`` cached keys, as
        (shares in a cluster, clusters per token and KV head): as many CTAs as are resident at once (two per
        SM), never more, so that no CTA waits for a second wave, and no share shorter than
        MIN_KEYS_PER_SPLIT keys.  Without a cluster kernel: (shares, 1)."""
        ctas = segments_count * self.shape.kv_heads * self.chunks
        n = max(1, min(MAX_SPLITS, (2 * self.sm_count) // ctas, max_positions // MIN_KEYS_PER_SPLIT))
        if self.clusters_of is None or self.chunks != 1 or n == 1:
            return n, 1
        # The shares of a cluster are merged in its shared memory, and a cluster is placed inside one
        # GPC: all the step's clusters must run at once (a second round of clusters costs more than
        # shorter shares gain).  The driver's count of resident clusters holds when nothing else is on
        # the GPU; the kernel before this one is still leaving, so large clusters, of which a GPC holds
        # two or three and has no room left, get two clusters of margin (measured at the 7B shape: 16
        # clusters of 13, of which 17 should fit, and 20 of 12, of which 21 should, took as long as two
        # rounds; 16 of 12, 20 and 24 of 10 and 32 of 8, of which 33 should fit, did not).  One or two
        # requests far into a long context have too few clusters of the largest size to keep the memory
        # busy: they get several clusters per token and KV head, whose parts attention_combine merges.
        # A launch is timed in the key tiles its longest CTA walks at the rate of a CTA that streams
        # alone; all CTAs together cannot walk more than some 240 tiles in that time (the memory's rate
        # over one CTA's), a CTA has a fixed cost, and parts left for attention_combine cost a launch and
        # a pass over them: several clusters per token must be a tenth faster by this count to be taken
        # (measured, 7B shape: one request at 32,000 keys 3.48 -> 3.18 ms a step with 8 clusters of 8;
        # two requests at 16,000 keys were no faster with 4 clusters of 8 than with one of 16).
        tiles = -(-max_positions // KEY_TILE)
        floor = ctas * tiles / self.STREAMS

        def cost(c, g):
            return max(-(-tiles // (c * g)), floor) + self.CTA_FIXED_TILES + (self.COMBINE_TILES if g > 1 else 0.0)

        def room(c):
            return self.clusters_of(c) - (2 if c > 10 else 0)

        best = None
        for c in range(min(n, self.max_cluster), 1, -1):
            if room(c) >= ctas:
                best = (c, 1)
                break
        if best is not None:
            best_cost = 0.9 * cost(*best)
            for c in range(min(n, self.max_cluster), 3, -1):
                for g in range(2, min(n // c, room(c) // ctas) + 1):
                    if cost(c, g) < best_cost:
                        best, best_cost = (c, g), cost(c, g)
        # no cluster fits: the shares go through the kernels that merge through global memory
        return best if best is not None else (n, 1)

    UNEVEN_CANDIDATES = (2, 3, 4, 6, 8, 12, 16)

    def decode_fixed_for(self, starts, max_positions):
        """More key splits than decode_fixed gives when the histories are uneven: with one CTA per token
        and KV head a batch waits for its longest history while most SMs have run out of work.  The
        duration of the launch is estimated by dealing its CTAs (each as long as its share of keys
        plus a fixed cost) to the resident slots in launch order, for decode_fixed's splits and for a
        few larger numbers; a larger number is only taken when it is a sixth faster, and the answer is
        remembered per rounded histories, so a captured graph is replaced seldom."""
        fixed = self.decode_fixed(len(starts), max_positions)
        n0 = fixed[0] * fixed[1]
        B = len(starts)
        limit = min(max_positions // MIN_KEYS_PER_SPLIT, self.max_cluster or MAX_SPLITS)
        if n0 > 1 or B < 2 or limit < 2:       # fewer requests: their splits are sized for one round of CTAs
            return fixed
        tiles = (np.asarray(starts, np.int64) + KEY_TILE) // KEY_TILE
        key = (n0, limit) + tuple(((tiles + 7) // 8).tolist())
        hit = self._uneven.get(key)
        if hit is not None:
            return hit
        ctas = B * self.shape.kv_heads * self.chunks
        best, best_time = n0, self._launch_time(tiles, n0)
        for n in self.UNEVEN_CANDIDATES:
            if n <= n0 or n > limit or ctas * n > 4096:
                continue
            t = self._launch_time(tiles, n)
            if t < best_time and t < self._launch_time(tiles, n0) / 1.2:
                best, best_time = n, t
        if len(self._uneven) > 512:
            self._uneven.clear()
        self._uneven[key] = (best, 1)
        return best, 1

    def _launch_time(self, tiles, n: int) -> float:
        """Key tiles of time until the last CTA of a decode launch with n key splits is done: CTAs start
        in launch order (splits of a token together, tokens in order, KV heads outermost) on two
        slots per SM, and a slot takes the next CTA when its own is done."""
        import heapq

        per_cta = np.repeat(-(-tiles // n) + self.CTA_FIXED_TILES, n)
        order = np.tile(per_cta, self.shape.kv_heads * self.chunks).tolist()
        slots = 2 * self.sm_count
        if len(order) <= slots:
            return max(order)
        busy = order[:slots]
        heapq.heapify(busy)
        for d in order[slots:]:
            heapq.heapreplace(busy, busy[0] + d)
        return max(busy)

    def plan_decode(self, starts, fixed):
        cluster, groups = fixed
        return self._out(plan_decode(self.shape, starts, cluster * groups), cluster if self.chunks == 1 else 0, groups)


@register_mixer("gq_attention")
class GQAttention(Mixer):
    """q/k/v projections (with bias), position encoding on q and k, append to the cache, causal
    grouped-query attention over the cache, output projection without bias
    (mini_hisparse/model.py:54-60, 135-153, 169-179, 157).

    Sizes are parameters: hidden_size, q_heads, kv_heads, head_dim, qkv_bias, window, and the
    position encoding's own spec.  Query head h reads KV head h // (q_heads // kv_heads).
    """

    def __init__(self, spec: PartSpec, rt=None):
        super().__init__(spec, rt)
        self.hidden = int(spec["hidden_size"])
        self.nq = int(spec["q_heads"])
        self.nkv = int(spec["kv_heads"])
        self.d = int(spec["head_dim"])
        self.qkv_bias = bool(spec.get("qkv_bias", True))
        self.window = spec.get("window")
        if self.nq % self.nkv:
            raise ValueError(f"{self.nq} query heads cannot be grouped over {self.nkv} KV heads")
        if self.d % 16 or not 16 <= self.d <= 256:
            raise ValueError(f"head_dim {self.d} is not supported: kernels take 16..256 in steps of 16")
        self.position = POSITIONS.build(spec["position"], rt=rt)
        self.scale = float(self.d) ** -0.5
        self.qkv_weight = self.qkv_bias_vec = self.o_weight = None

    @property
    def tensor_core_attention(self) -> bool:
        """bfloat16 and a head size the mma kernel is built for; else the CUDA-core kernel."""
        return (self.rt is not None and self.rt.dtype == torch.bfloat16 and self.d in K.MMA_HEAD_DIMS)

    def kernel_family(self, page_size: int) -> str:
        """Which attention kernels serve pages of ``page_size`` keys: "tc" (TMA-fed 16-row tiles for
        short segments, tcgen05 128-row tiles for long portions: bfloat16, head size 64 or 128,
        pages that divide 64), "mma" (mma.sync with 16- and 64-row tiles: bfloat16, head size 32,
        64, 96 or 128, any page size) or "simt" (CUDA cores: everything else)."""
        if not self.tensor_core_attention:
            return "simt"
        return "tc" if K.attention_tma_supports(self.d, page_size) else "mma"

    def big_tile_rows(self, page_size: int) -> int:
        """Query rows per tile for long portions."""
        return {"tc": 128, "mma": 64, "simt": ROW_TILE}[self.kernel_family(page_size)]

    def kernel_modules(self):
        """attention_simt holds the CUDA-core kernel and the merge of key splits; the tensor-core
        kernels come in for the head sizes they are built for (which of them runs depends on the
        page size, which the cache brings)."""
        if not self.tensor_core_attention:
            return ("attention_simt",)
        if self.d in (64, 128):
            return ("attention_simt", "attention_mma", "attention_tma", "attention_decode", "attention_tc")
        return ("attention_simt", "attention_mma")

    def cache_need(self):
        return PagedKVNeed(kv_heads=self.nkv, head_dim=self.d, window=self.window)

    def plan_key(self):
        return ("gq_attention", self.nq, self.nkv, self.d, self.window)

    def planner(self, page_size: int, sm_count: int):
        shape = AttentionShape(self.nq, self.nkv, self.window, self.big_tile_rows(page_size))
        if self.kernel_family(page_size) == "tc" and self.nq // self.nkv <= ROW_TILE:
            return AttentionPlanner(shape, sm_count, lambda n: K.attention_decode_max_clusters(self.d, n),
                                    K.DECODE_MAX_SPLITS)
        return AttentionPlanner(shape, sm_count)

    def parameters(self):
        q, kv = self.nq * self.d, self.nkv * self.d
        p = {
            "q_proj.weight": ParamSpec((q, self.hidden)),
            "k_proj.weight": ParamSpec((kv, self.hidden)),
            "v_proj.weight": ParamSpec((kv, self.hidden)),
            "o_proj.weight": ParamSpec((self.hidden, q)),
        }
        if self.qkv_bias:
            p["q_proj.bias"] = ParamSpec((q,), role="vector")
            p["k_proj.bias"] = ParamSpec((kv,), role="vector")
            p["v_proj.bias"] = ParamSpec((kv,), role="vector")
        return p

    def load(self, tensors):
        self.qkv_weight = torch.cat(
            (tensors["q_proj.weight"], tensors["k_proj.weight"], tensors["v_proj.weight"]), 0
        ).contiguous()
        if self.qkv_bias:
            self.qkv_bias_vec = torch.cat(
                (tensors["q_proj.bias"], tensors["k_proj.bias"], tensors["v_proj.bias"]), 0
            ).contiguous()
        self.o_weight = tensors["o_proj.weight"].contiguous()

    def forward(self, h, ctx: StepContext, cache: CacheView) -> Product:
        rt, ws, T = ctx.rt, ctx.ws, h.shape[0]
        meta = cache.meta
        family = self.kernel_family(cache.page_size)
        rdim = int(getattr(self.position, "rotary_dim", 0) or 0)
        interleaved = bool(getattr(self.position, "interleaved", False))
        nsplit, ngroups = meta.get("decode_nsplit", 0), meta.get("decode_groups", 1)
        if (family == "tc" and nsplit and cache.writable
                and K.attention_decode_supports(self.d, cache.page_size, self.nq // self.nkv, nsplit, rdim)):
            # single new tokens only: sum of the product's parts, bias, rotation, append, attention and
            # the merge of the key splits are one kernel
            qkv = rt.linear(h, self.qkv_weight, ws, "qkv", out_dtype=torch.float32)
            attn = ws.get("attn", (T, self.nq * self.d), rt.dtype)
            parts = {}
            if ngroups > 1:         # several clusters per token and KV head leave a part each
                parts = dict(ngroups=ngroups,
                             part_acc=ws.get("attn_part_acc", (T * ngroups, self.nq, self.d), torch.float32),
                             part_ml=ws.get("attn_part_ml", (T * ngroups, self.nq, 2), torch.float32))
            K.attention_decode(qkv.tensor, self.qkv_bias_vec, self.position.inv_freq, cache.storage, attn,
                               ctx.positions, meta["block_table"], nq=self.nq, nkv=self.nkv, d=self.d,
                               page_size=cache.page_size, nsplit=nsplit, qkv_nsplit=qkv.nsplit,
                               qkv_split_stride=qkv.split_stride, rotary_dim=rdim, interleaved=interleaved,
                               window=self.window or 0, scale=self.scale, status=ctx.status, **parts)
            return rt.linear(attn, self.o_weight, ws, "mix_out")
        q = ws.get("q", (T, self.nq * self.d), rt.dtype)
        fused = rt.qkv_rope_append(h, self.qkv_weight, self.qkv_bias_vec, ctx, self.position, meta["block_table"],
                                   q, cache.storage, nq=self.nq, nkv=self.nkv, d=self.d,
                                   page_size=cache.page_size, write_kv=cache.writable)
        if not fused:
            qkv = rt.linear(h, self.qkv_weight, ws, "qkv", out_dtype=torch.float32)
            K.rope_append(
                qkv.tensor, self.qkv_bias_vec, ctx.positions, ctx.tok_seg, meta["block_table"],
                self.position.inv_freq, q, cache.storage, nq=self.nq, nkv=self.nkv, d=self.d,
                page_size=cache.page_size, write_kv=cache.writable, rotary_dim=rdim, interleaved=interleaved,
                nsplit=qkv.nsplit, split_stride=qkv.split_stride, status=ctx.status,
            )
        attn = ws.get("attn", (T, self.nq * self.d), rt.dtype)
        part_rows = max(1, meta["part_rows_cap"])
        part_acc = ws.get("attn_part_acc", (part_rows, self.nq, self.d), torch.float32)
        part_ml = ws.get("attn_part_ml", (part_rows, self.nq, 2), torch.float32)
        common = dict(nq=self.nq, nkv=self.nkv, d=self.d, page_size=cache.page_size,
                      window=self.window or 0, scale=self.scale)
        args = (q, cache.storage, attn, part_acc, part_ml)
        tail = (ctx.positions, meta["block_table"], meta["tok_part_row"])
        n_small, n_big = meta["n_small"], meta["n_big"]
        if family != "simt":
            tma = family == "tc"
            kernel = K.attention_tma if tma else K.attention_mma
            extra = {"status": ctx.status} if tma else {}
            def short_segments():
                chunks = -(-(self.nq // self.nkv) // ROW_TILE)
                counters = ws.get_zeroed("attn_counters", (T * self.nkv * chunks,), torch.int32)
                # short segments have at most SPLIT_MAX_TOKENS tokens: only the keys that close to a
                # token's position can come from this step's append, the kernel launched just before
                fresh = {"fresh": SPLIT_MAX_TOKENS} if tma else {}
                kernel(*args, meta["items"], n_small, 16, *tail, **common, **extra, **fresh,
                       tok_nsplit=meta["tok_nsplit"], counters=counters)

            def long_portions():
                big_items = meta["items"][n_small * ITEM_INTS:]
                if tma:
                    K.attention_tc(q, cache.storage, attn, big_items, n_big, ctx.positions, meta["block_table"],
                                   part_acc=part_acc, part_ml=part_ml, tok_part_row=meta["tok_part_row"],
                                   status=ctx.status, **common)
                    if meta.get("big_split"):
                        K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], attn,
                                            nq=self.nq, d=self.d)
                else:
                    kernel(*args, big_items, n_big, 64, *tail, **common, **extra)

            side = ctx.extras.get("side_stream") if (n_small >= 8 and n_big >= 8 and not meta.get("big_split")) else None
            if side is not None:
                # The two kernels touch different tokens: the long portions run on a second stream beside
                # the short segments (a mixed serving step has some dozens of decode tokens beside a
                # prompt portion, and neither kernel fills the GPU for as long as the other runs).
                ctx.extras["two_stream_layers"] = ctx.extras.get("two_stream_layers", 0) + 1
                main = torch.cuda.current_stream()
                fork, join = ctx.extras["side_events"]
                fork.record(main)
                side.wait_event(fork)
                with torch.cuda.stream(side), K.stream_scope():
                    long_portions()
                    join.record(side)
                short_segments()
                main.wait_event(join)
            else:
                if n_small:
                    short_segments()
                if n_big:
                    long_portions()
        elif n_small + n_big:
            K.attention_simt(*args, meta["items"], n_small + n_big, n_small + n_big, *tail, **common)
        if meta["any_split"] and family == "simt":
            K.attention_combine(part_acc, part_ml, meta["tok_part_row"], meta["tok_nsplit"], attn,
                                nq=self.nq, d=self.d)
        return rt.linear(attn, self.o_weight, ws, "mix_out")
