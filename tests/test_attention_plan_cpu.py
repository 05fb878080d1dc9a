"""The attention plan (host only): whatever the mix of segments, every (token, query head, key) that
causal attention needs is covered by exactly one work item, parts of a split tile are numbered
0..n-1 and own distinct partial rows, and capacity bounds hold."""
import numpy as np
import pytest

from mini_hisparse_b200.parts.attention import (ITEM_INTS, MAX_SPLITS, ROW_TILE, plan_attention, plan_capacity,
                                                plan_decode)
from mini_hisparse_b200.parts.base import Segment
from mini_hisparse_b200.parts.attention import AttentionShape


def segments_of(specs):
    """specs: (cached tokens, new tokens) per request."""
    out, off = [], 0
    for i, (hist, n) in enumerate(specs):
        out.append(Segment(f"r{i}", i, hist, n, off))
        off += n
    return out, off


def check_cover(need, specs, plan):
    segments, T = segments_of(specs)
    groups = need.q_heads // need.kv_heads
    window = need.window or 0
    pos = np.concatenate([np.arange(h, h + n) for h, n in specs])
    covered = {}                                  # (token, head in group) -> list of (begin, end, split)
    for it in plan.items:
        si, tok0, nt, h0, nh, b, e, sp = (int(v) for v in it)
        seg = segments[si]
        assert seg.offset <= tok0 and tok0 + nt <= seg.offset + seg.count
        assert 0 <= h0 and h0 + nh <= groups and nt * nh <= max(ROW_TILE, need.tile_rows)
        for t in range(tok0, tok0 + nt):
            for h in range(h0, h0 + nh):
                covered.setdefault((t, h), []).append((b, e, sp))
    assert len(covered) == T * groups             # every token and head has items
    for (t, h), parts in covered.items():
        lo = max(0, int(pos[t]) - window + 1) if window else 0
        hi = int(pos[t]) + 1                      # keys [lo, hi) are what the token may see
        parts.sort()
        splits = [p[2] for p in parts]
        if len(parts) == 1 and splits[0] < 0:
            assert plan.tok_nsplit[t] == 0
        else:
            assert sorted(splits) == list(range(len(parts))) == list(range(int(plan.tok_nsplit[t])))
        # the parts tile a range that contains [lo, hi) without gap or overlap (the kernels mask
        # per token inside an item, so an item may reach beyond a token's own range)
        for (b0, e0, _), (b1, e1, _) in zip(parts, parts[1:]):
            assert e0 == b1 or e0 >= hi           # later parts may be empty past the end
        assert parts[0][0] <= lo and max(p[1] for p in parts) >= hi
    # partial rows: each split token owns tok_nsplit consecutive rows, nobody shares
    rows = set()
    for t in range(T):
        n = int(plan.tok_nsplit[t])
        assert n <= MAX_SPLITS                    # what the attention kernels' merge has scratch for
        for r in range(int(plan.tok_part_row[t]), int(plan.tok_part_row[t]) + n):
            assert r not in rows and r < plan.part_rows
            rows.add(r)
    assert plan.n_small + plan.n_big == plan.items.shape[0]


CASES = [
    [(0, 300), (45, 19), (130, 1), (200, 170), (0, 1), (77, 129)],
    [(3000, 100), (2500, 1), (700, 1), (1800, 40)],
    [(4000, 1)] * 8,
    [(100 + 61 * i, 1) for i in range(30)] + [(3000, 482)],
    [(0, 2048)],
    [(16000, 100)],
    [(0, 1), (0, 2), (0, 16), (0, 17)],
]


@pytest.mark.parametrize("specs", CASES)
@pytest.mark.parametrize("need", [
    AttentionShape(28, 4, None, 128), AttentionShape(40, 8, None, 128),
    AttentionShape(3, 1, None, 64), AttentionShape(4, 2, None, 16),
    AttentionShape(512, 2, None, 128), AttentionShape(4, 4, 100, 128),
])
def test_every_key_is_covered_once(need, specs):
    segments, T = segments_of(specs)
    plan = plan_attention(need, segments, T, 148)
    check_cover(need, specs, plan)
    items, rows = plan_capacity(need, T, len(specs))
    assert plan.items.shape[0] <= items and plan.part_rows <= rows


def test_long_tiles_are_split_only_when_they_are_fewer_than_sms():
    need = AttentionShape(28, 4, None, 128)
    few = plan_attention(need, segments_of([(16000, 100)])[0], 100, 148)
    assert few.big_split and (few.items[few.n_small:, 7] >= 0).all()
    many = plan_attention(need, segments_of([(0, 2048)])[0], 2048, 148)
    assert not many.big_split and (many.items[:, 7] == -1).all()
    spans = many.items[:, 6] - many.items[:, 5]
    assert (np.diff(spans) <= 0).all()            # longest tiles first


def test_a_long_history_beside_short_ones_gets_more_parts():
    need = AttentionShape(40, 8, None, 128)
    specs = [(4000, 1)] + [(200, 1)] * 29
    plan = plan_attention(need, segments_of(specs)[0], 30, 148)
    assert plan.tok_nsplit[0] >= 2 and (plan.tok_nsplit[1:] <= 1).all()
    assert plan.tok_nsplit.max() <= MAX_SPLITS


@pytest.mark.parametrize("nsplit", [1, 3, 16])
def test_decode_plan_for_a_captured_graph(nsplit):
    need = AttentionShape(28, 4, None, 128)
    starts = np.array([4000, 17, 0, 999], np.int64)
    plan = plan_decode(need, starts, nsplit)
    assert plan.items.shape == (4 * nsplit, ITEM_INTS)
    assert plan.part_rows == (4 * nsplit if nsplit > 1 else 0)
    check_cover(need, [(int(s), 1) for s in starts], plan)


def test_uneven_histories_get_more_key_splits_than_even_ones():
    """A decode batch that fills the GPU with one CTA per token and KV head waits for its longest
    history; the planner then cuts every token's keys into a few parts (the same number for all: a
    captured graph has a fixed launch size).  Even histories keep what decode_fixed gives, the answer
    does not change from step to step, and the plan with more parts still covers every key once."""
    from mini_hisparse_b200.parts.attention import AttentionPlanner

    resident = {1: 296, 2: 148, 3: 98, 4: 74, 5: 59, 6: 49, 7: 42, 8: 33, 9: 30, 10: 24, 11: 24, 12: 20, 13: 20,
                14: 20, 15: 16, 16: 16}
    need = AttentionShape(40, 8, None, 128)
    planner = AttentionPlanner(need, 148, lambda n: resident[n], 16)
    uneven = np.random.default_rng(1).integers(128, 4224, 29)
    base = planner.decode_fixed(29, 8192)
    more = planner.decode_fixed_for(uneven, 8192)
    assert base == (1, 1) and 2 <= more[0] <= 16 and more[1] == 1
    assert planner._launch_time((uneven + 64) // 64, more[0]) < planner._launch_time((uneven + 64) // 64, 1) / 1.2
    assert all(planner.decode_fixed_for(uneven + step, 8192) == more for step in range(1, 40))
    arrays, facts = planner.plan_decode(uneven, more)
    assert facts["decode_nsplit"] == more[0] and facts["decode_groups"] == 1
    check_cover(need, [(int(s), 1) for s in uneven], plan_decode(need, uneven, more[0]))
    for B in (1, 2, 8, 16, 32, 64):        # even histories: nothing to gain
        even = np.full(B, 4095)
        small = AttentionPlanner(AttentionShape(28, 4, None, 128), 148, lambda n: resident[n], 16)
        assert small.decode_fixed_for(even, 4096) == small.decode_fixed(B, 4096)


def test_cluster_sizes_of_a_decode_step():
    """decode_fixed with the resident-cluster counts that the driver reports for the decode kernel on a
    B200 (two CTAs per SM): the largest cluster of which all of a step's clusters run at once, with
    two clusters to spare above ten CTAs a cluster, and never more splits than the largest cluster
    when the fused launch's shares are at most four times longer."""
    from mini_hisparse_b200.parts.attention import AttentionPlanner

    reported = {1: 296, 2: 148, 3: 93, 4: 71, 5: 56, 6: 45, 7: 37, 8: 33, 9: 30, 10: 26, 11: 21, 12: 21, 13: 17,
                14: 14, 15: 14, 16: 14}
    planner = AttentionPlanner(AttentionShape(28, 4, None, 128), 148, lambda n: reported[n], 16)
    assert [planner.decode_fixed(B, 4096) for B in (1, 2, 3, 4, 5, 6, 8, 16, 32, 64)] == [
        (16, 1), (16, 1), (16, 1), (12, 1), (10, 1), (10, 1), (8, 1), (4, 1), (2, 1), (1, 1)]
    # one request far into a long context: several clusters per KV head, all resident at once
    cluster, groups = planner.decode_fixed(1, 32768)
    assert groups > 1 and 48 <= cluster * groups <= 64 and reported[cluster] >= 4 * groups + (2 if cluster > 10 else 0)
    assert planner.decode_fixed(1, 8192) == (16, 1)      # a second launch to merge parts would cost more than it saves
    cluster, groups = planner.decode_fixed(4, 32768)
    assert cluster * groups <= 18 and reported[cluster] >= 16 * groups + (2 if cluster > 10 else 0)
    assert planner.decode_fixed(8, 512) == (2, 1)        # no share shorter than 256 keys
    arrays, facts = planner.plan_decode(np.array([32000]), planner.decode_fixed(1, 32768))
    cluster, groups = planner.decode_fixed(1, 32768)
    assert facts["decode_nsplit"] == cluster and facts["decode_groups"] == groups
    assert len(arrays["items"]) == cluster * groups * ITEM_INTS
    plain = AttentionPlanner(AttentionShape(28, 4, None, 128), 148)      # a kernel without clusters
    assert plain.decode_fixed(1, 32768) == (64, 1) and plain.decode_fixed(4, 4096) == (16, 1)
