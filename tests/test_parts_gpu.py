"""Each part alone on the GPU against its plain formula: norm, position encoding inside the
mixer, attention mixer over its own cache, feed-forward, embedding and head, and a whole block."""
import pytest
import torch

from conftest import random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def harness(needs, dtype, num_pages=16, page_size=16):
    from mini_hisparse_b200 import CacheConfig, CacheManager
    from mini_hisparse_b200.engine.step import BatchBuilder
    from mini_hisparse_b200.kernels.runtime import make_runtime
    from mini_hisparse_b200.parts import Workspace

    rt = make_runtime(DEV, dtype)
    cache = CacheManager(needs, CacheConfig(num_pages=num_pages, page_size=page_size, max_requests=4,
                                            dtype=dtype, device=DEV))
    return rt, cache, BatchBuilder(cache, DEV), Workspace(DEV), torch.zeros(1, dtype=torch.int32, device=DEV)


def context(rt, cache, batch, ws, status, entries):
    segments, T = batch.segments(entries)
    for s in segments:
        cache.ensure(s.request, s.start + s.count)
    views = batch.eager(entries, segments)
    return batch.context(rt, ws, status, views, segments), views, segments


def fill(part, seed, dtype, std=0.2):
    from mini_hisparse_b200.weights.loader import draw

    tensors, plain = {}, {}
    for name, ps in part.parameters().items():
        t = draw(name, ps, seed, matrix_std=std).to(torch.bfloat16).float()   # bf16-exact values
        plain[name] = t
        tensors[name] = t.to(DEV, torch.float32 if ps.role == "vector" else dtype)
    part.load(tensors)
    return plain


def tol(dtype, ref):
    if dtype == torch.float32:
        return dict(atol=2e-5 * max(1.0, float(ref.abs().max())), rtol=2e-5)
    return dict(atol=0.02 * float(ref.abs().max()), rtol=0.02)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_part(dtype):
    from mini_hisparse_b200.engine import StepEntry
    from mini_hisparse_b200.parts import NORMS, PartSpec, Product

    rt, cache, batch, ws, status = harness([], dtype)
    norm = NORMS.build(PartSpec.make("rmsnorm", width=200, eps=1e-4), rt=rt)
    w = fill(norm, 1, dtype)
    cache.open("a")
    ctx, _, _ = context(rt, cache, batch, ws, status, [StepEntry("a", [1] * 9, [])])
    x = torch.randn(9, 200, device=DEV)
    delta = torch.randn(9, 200, device=DEV).to(dtype)
    x0 = x.clone()
    out = norm.forward(x, ctx, delta=Product(delta))
    torch.testing.assert_close(x, x0 + delta.float())
    ref = P.rms_norm((x0 + delta.float()).cpu(), w["weight"], 1e-4)
    torch.testing.assert_close(out.float().cpu(), ref, **tol(dtype, ref))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("nq,nkv,d,theta", [(6, 2, 32, 1e4), (5, 5, 16, 1e6), (8, 1, 64, 500.0)])
def test_attention_mixer_over_its_cache(dtype, nq, nkv, d, theta):
    """Prompt in two portions and three decoded tokens, two requests interleaved."""
    from mini_hisparse_b200.engine import StepEntry
    from mini_hisparse_b200.parts import MIXERS, PartSpec

    H = 72
    spec = PartSpec.make("gq_attention", hidden_size=H, q_heads=nq, kv_heads=nkv, head_dim=d, qkv_bias=True,
                         window=None, position=PartSpec.make("rotary", head_dim=d, theta=theta))
    rt, cache, batch, ws, status = harness([MIXERS.get("gq_attention")(spec).cache_need()], dtype)
    mixer = MIXERS.build(spec, rt=rt)
    user = batch.add_user(0, mixer)      # the mixer's planner joins the step's packing
    w = fill(mixer, 2, dtype)

    @dataclass_like
    class Cfg:
        num_attention_heads, num_key_value_heads, head_dim, rope_theta = nq, nkv, d, theta

    hs = {r: torch.randn(n, H, generator=torch.Generator().manual_seed(i)).to(torch.bfloat16).float()
          for i, (r, n) in enumerate({"a": 45, "b": 23}.items())}
    refs = {r: P.attention_block(Cfg, {"x." + k: v for k, v in w.items()}, "x.", h, torch.arange(len(h)))
            for r, h in hs.items()}
    cuts = {"a": [30, 12, 1, 1, 1], "b": [1, 1, 19, 1, 1]}
    done = {"a": 0, "b": 0}
    cache.open("a"), cache.open("b")
    for step in range(5):
        entries = [StepEntry(r, [0] * cuts[r][step], []) for r in ("a", "b")]
        ctx, views, segments = context(rt, cache, batch, ws, status, entries)
        h = torch.cat([hs[r][done[r]: done[r] + cuts[r][step]] for r in ("a", "b")]).to(DEV, dtype)
        out = mixer.forward(h, ctx, batch.cache_view(user, views)).reduced().cpu()
        row = 0
        for r in ("a", "b"):
            n = cuts[r][step]
            ref = refs[r][done[r]: done[r] + n]
            torch.testing.assert_close(out[row: row + n], ref, **tol(dtype, refs[r]))
            row += n
            done[r] += n
            cache.advance(r, n)
    assert int(status) == 0


def dataclass_like(cls):
    return cls


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu_embedding_head_parts(dtype):
    from mini_hisparse_b200.engine import StepEntry
    from mini_hisparse_b200.parts import EMBEDDINGS, FEED_FORWARDS, HEADS, PartSpec

    rt, cache, batch, ws, status = harness([], dtype)
    cache.open("a")
    tokens = random_tokens(333, 11, 4)
    ctx, _, _ = context(rt, cache, batch, ws, status, [StepEntry("a", tokens, [])])
    ff = FEED_FORWARDS.build(PartSpec.make("swiglu", hidden_size=88, intermediate_size=200), rt=rt)
    w = fill(ff, 3, dtype)
    h = torch.randn(11, 88).to(torch.bfloat16).float()
    out = ff.forward(h.to(DEV, dtype), ctx).reduced().cpu()
    ref = P.swiglu(h, w["gate_proj.weight"], w["up_proj.weight"], w["down_proj.weight"])
    torch.testing.assert_close(out, ref, **tol(dtype, ref))

    emb = EMBEDDINGS.build(PartSpec.make("token_embedding", vocab_size=333, hidden_size=88), rt=rt)
    we = fill(emb, 4, dtype)
    x = emb.forward(ctx)
    assert x.dtype == torch.float32
    torch.testing.assert_close(x.cpu(), we["weight"][torch.tensor(tokens)])
    head = HEADS.build(PartSpec.make("lm_head", vocab_size=333, hidden_size=88, tied=True), rt=rt)
    head.load({})
    head.tie(emb)
    logits = head.forward(h.to(DEV, dtype), ctx)
    assert logits.dtype == torch.float32
    ref = h @ we["weight"].T
    torch.testing.assert_close(logits.cpu(), ref, **tol(dtype, ref))


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_block_alone(dtype, folders):
    """One pre-norm block of Tiny B's shape: the pending output of a previous block goes in, the
    block's own unadded output comes out."""
    from conftest import TINY_B
    from mini_hisparse_b200 import resolve
    from mini_hisparse_b200.engine import StepEntry
    from mini_hisparse_b200.parts import BLOCKS, Product

    cfg, spec = resolve(TINY_B)
    layer = spec.layers[1]
    block0 = BLOCKS.get(layer.block)(layer, None)
    rt, cache, batch, ws, status = harness([block0.cache_need()], dtype, page_size=32)
    block = BLOCKS.get(layer.block)(layer, rt)
    user = batch.add_user(0, block)
    pw, sd = P.load_folder(folders["B"])
    for role, part in block.parts().items():
        prefix = f"{layer.prefix}.{layer.name_of(role)}."
        part.load({k: sd[prefix + k].to(DEV, torch.float32 if ps.role == "vector" else dtype)
                   for k, ps in part.parameters().items()})
    cache.open("a")
    T = 40
    ctx, views, _ = context(rt, cache, batch, ws, status, [StepEntry("a", [0] * T, [])])
    x0 = torch.randn(T, 96)
    pend = (torch.randn(T, 96) * 0.3).to(torch.bfloat16).float()
    x = x0.clone().to(DEV)
    out = block.forward(x, Product(pend.to(DEV, dtype)), ctx, batch.cache_view(user, views))
    total = x.cpu() + out.reduced().cpu()
    ref = P.decoder_layer(pw, sd, 1, x0 + pend, torch.arange(T))
    torch.testing.assert_close(total, ref, **tol(dtype, ref))
