"""The plain implementation against the reference's own model code (golden files) and against
simple properties of its parts.  No GPU."""
import json
from pathlib import Path

import numpy as np
import torch

from plain import qwen2_plain as P

GOLD = Path(__file__).parent / "golden" / "tiny_ref"


def _gold():
    meta = json.loads((GOLD / "golden.json").read_text())
    logits = torch.from_numpy(
        np.fromfile(GOLD / "prefix_logits.f32", dtype="<f4").reshape(meta["logits_shape"]).copy()
    )
    return meta, logits


def test_plain_logits_equal_reference_model_code():
    """tests/test_engine.py:101 of the reference compares at atol 2e-6, rtol 2e-5."""
    meta, gold = _gold()
    cfg, w = P.load_folder(GOLD)
    ours = P.forward_logits(cfg, w, meta["tokens"])
    torch.testing.assert_close(ours, gold, atol=2e-6, rtol=2e-5)


def test_plain_greedy_equals_reference_engine():
    meta, _ = _gold()
    cfg, w = P.load_folder(GOLD)
    for name, prompt in meta["prompts"].items():
        assert P.generate(cfg, w, prompt, len(meta["greedy"][name])) == meta["greedy"][name]


def test_rows_do_not_depend_on_later_tokens():
    cfg, w = P.load_folder(GOLD)
    toks = list(range(3, 33))
    full = P.forward_logits(cfg, w, toks)
    part = P.forward_logits(cfg, w, toks[:11])
    torch.testing.assert_close(full[:11], part, atol=1e-6, rtol=1e-5)


def test_attention_is_causal_grouped_and_windowed():
    torch.manual_seed(0)
    T, nq, nkv, d = 9, 4, 2, 8
    q, k, v = torch.randn(T, nq, d), torch.randn(T, nkv, d), torch.randn(T, nkv, d)
    out = P.causal_attention(q, k, v)
    for t in range(T):
        for h in range(nq):
            kh = h // (nq // nkv)
            s = (k[: t + 1, kh] @ q[t, h]) / d ** 0.5
            ref = s.softmax(0) @ v[: t + 1, kh]
            torch.testing.assert_close(out[t, h], ref, atol=1e-6, rtol=1e-5)
    win = P.causal_attention(q, k, v, window=3)
    t, h = 7, 1
    s = (k[5:8, 0] @ q[t, h]) / d ** 0.5
    torch.testing.assert_close(win[t, h], s.softmax(0) @ v[5:8, 0], atol=1e-6, rtol=1e-5)


def test_rotation_keeps_norm_and_is_relative():
    pos = torch.arange(50)
    cos, sin = P.rope_tables(pos, 16, 10000.0, torch.float32)
    x = torch.randn(50, 3, 16)
    r = P.rotate(x, cos, sin)
    torch.testing.assert_close(r.norm(dim=-1), x.norm(dim=-1), atol=1e-5, rtol=1e-5)
    # the score of a rotated pair depends on the distance only
    q, k = torch.randn(16), torch.randn(16)
    def score(pq, pk):
        c, s = P.rope_tables(torch.tensor([pq, pk]), 16, 10000.0, torch.float32)
        a = P.rotate(torch.stack((q, k))[:, None], c, s)
        return float(a[0, 0] @ a[1, 0])
    assert abs(score(7, 3) - score(27, 23)) < 1e-4


def test_rms_norm_and_swiglu_formulas():
    x = torch.randn(5, 12)
    wt = torch.rand(12) + 0.5
    y = P.rms_norm(x, wt, 1e-5)
    ref = x / torch.sqrt((x * x).mean(-1, keepdim=True) + 1e-5) * wt
    torch.testing.assert_close(y, ref, atol=1e-6, rtol=1e-5)
    g, u, dn = torch.randn(7, 12), torch.randn(7, 12), torch.randn(12, 7)
    out = P.swiglu(x, g, u, dn)
    a = x @ g.T
    ref = ((a / (1 + torch.exp(-a))) * (x @ u.T)) @ dn.T
    torch.testing.assert_close(out, ref, atol=1e-5, rtol=1e-5)


def test_sampling_draw():
    us = [P.uniform_from_counter(5, i) for i in range(2000)]
    assert all(0.0 <= u < 1.0 for u in us) and 0.45 < sum(us) / len(us) < 0.55
    assert P.uniform_from_counter(5, 1) != P.uniform_from_counter(6, 1)
    logits = torch.tensor([0.0, 1.0, 2.0, -1.0])
    counts = [0] * 4
    for i in range(4000):
        counts[P.sample_temperature(logits, 0.7, 3, i)[0]] += 1
    p = (logits / 0.7).softmax(0)
    for c, pi in zip(counts, p.tolist()):
        assert abs(c / 4000 - pi) < 0.03
    assert P.greedy(torch.tensor([1.0, 3.0, 3.0])) == 1
