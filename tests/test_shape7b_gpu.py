"""The layer sizes of the benchmark (Qwen2.5-7B: hidden 3584, 28 query heads over 4 KV heads of 128,
feed-forward 18944) with two layers and a smaller vocabulary that is no power of two: the kernels
at the sizes they are tuned for, in float32 and in bfloat16, whole prompt, portions and decode,
against the plain implementation run in float32 on the device."""
import json

import numpy as np
import pytest
import torch

from conftest import random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

CONFIG = dict(
    architectures=["Qwen2ForCausalLM"], model_type="qwen2", vocab_size=30011, hidden_size=3584,
    intermediate_size=18944, num_hidden_layers=2, num_attention_heads=28, num_key_value_heads=4,
    rms_norm_eps=1e-6, rope_theta=1000000.0, tie_word_embeddings=False, max_position_embeddings=4096,
)


@pytest.fixture(scope="module")
def folder(tmp_path_factory):
    """Weights drawn on the GPU (fast) and written through the package's safetensors writer."""
    from mini_hisparse_b200 import resolve
    from mini_hisparse_b200.weights import write_safetensors
    from mini_hisparse_b200.weights.expected import expected_tensors_of_spec

    out = tmp_path_factory.mktemp("shape7b")
    gen = torch.Generator(device="cuda:0").manual_seed(77)
    tensors = {}
    for name, ps in expected_tensors_of_spec(resolve(CONFIG)[1]).items():
        mean, std = (1.0, 0.1) if "norm" in name else (0.0, 0.02)
        if ps.role == "matrix":
            std = 1.5 / (ps.shape[-1] ** 0.5)       # activations of order one: attention is not uniform
        t = torch.empty(ps.shape, device="cuda:0").normal_(mean, std, generator=gen)
        tensors[name] = (t.bfloat16() if ps.role == "matrix" else t).cpu()
    (out / "config.json").write_text(json.dumps(CONFIG))
    write_safetensors(out / "model.safetensors", tensors)
    return out


@pytest.fixture(scope="module")
def reference(folder):
    torch.backends.cuda.matmul.allow_tf32 = False
    torch.backends.cudnn.allow_tf32 = False
    cfg, w = P.load_folder(folder, dtype=torch.float32, device="cuda:0")
    tokens = random_tokens(CONFIG["vocab_size"], 700, seed=9)
    return tokens, P.forward_logits(cfg, w, tokens).cpu()


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_7b_layer_sizes_all_cuts(folder, reference, dtype):
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    tokens, ref = reference
    model = load_model(folder, dtype=dtype)
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=96, page_size=16, max_requests=4,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    tol = dict(atol=1e-3, rtol=1e-3) if dtype == "float32" else dict(atol=0.03 * float(ref.abs().max()), rtol=0.03)

    def run(name, cuts):
        cache.open(name)
        rows, i = [], 0
        for n in cuts:
            out = runner.step([StepEntry(name, tokens[i:i + n], list(range(n)))])
            rows.append(out.float().cpu().clone())
            i += n
        runner.check_status()
        cache.close(name)
        return torch.cat(rows), i

    got, n = run("whole", [700])
    torch.testing.assert_close(got, ref[:n], **tol)
    got, n = run("portions", [300, 65, 2, 130, 17, 2] + [1] * 20)       # the ones go through a graph
    torch.testing.assert_close(got, ref[:n], **tol)
    if dtype == "bfloat16":
        agree = (got.argmax(-1) == ref[:n].argmax(-1)).float().mean()
        assert agree > 0.9
    assert runner.stats["graph_steps"] >= 20
    cache.assert_invariants()


def test_7b_layer_sizes_long_prompt_shares_tiles_along_k(folder):
    """1,400 tokens in one step, bfloat16: the down projection (K = 18944) has 11 x 14 = 154 tiles for
    148 SMs, so the persistent product cuts the six tiles of its last round along K into eight parts
    each and reduces them through the workspace; the prompt also spans 22 key tiles in the tcgen05
    attention kernel."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    torch.backends.cuda.matmul.allow_tf32 = False
    cfg, w = P.load_folder(folder, dtype=torch.float32, device="cuda:0")
    tokens = random_tokens(CONFIG["vocab_size"], 1400, seed=11)
    want = list(range(0, 1400, 7)) + [1399]
    ref = P.forward_logits(cfg, w, tokens)[want].cpu()
    model = load_model(folder, dtype="bfloat16")
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=160, page_size=16, max_requests=2,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    cache.open("long")
    outs = []
    for _ in range(2):          # twice: the workspace counters are back at zero after a step
        cache.close("long")
        cache.open("long")
        outs.append(runner.step([StepEntry("long", tokens, want)]).float().cpu().clone())
    runner.check_status()
    assert int(model.rt.scratch()[1].abs().sum()) == 0
    assert torch.equal(outs[0], outs[1])
    torch.testing.assert_close(outs[0], ref, atol=0.03 * float(ref.abs().max()), rtol=0.03)
    assert (outs[0].argmax(-1) == ref.argmax(-1)).float().mean() > 0.9
    cache.assert_invariants()


def test_7b_layer_sizes_decode_tokens_beside_a_long_portion(folder):
    """One step with eight decode tokens and a 300-token portion, bfloat16: the attention of the long
    portion (tcgen05 kernel) runs on a second stream beside the attention of the decode tokens; every
    row is compared with the plain implementation of its own request."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    torch.backends.cuda.matmul.allow_tf32 = False
    cfg, w = P.load_folder(folder, dtype=torch.float32, device="cuda:0")
    model = load_model(folder, dtype="bfloat16")
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=120, page_size=16, max_requests=10,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    short = [random_tokens(CONFIG["vocab_size"], 20 + 9 * i, seed=30 + i) for i in range(8)]
    long_prompt = random_tokens(CONFIG["vocab_size"], 420, seed=50)
    for i, toks in enumerate(short):                       # prefill all but the last token of the short ones
        cache.open(f"s{i}")
        runner.step([StepEntry(f"s{i}", toks[:-1], [])])
    cache.open("long")
    runner.step([StepEntry("long", long_prompt[:120], [])])
    assert runner.stats["two_stream_layers"] == 0
    entries = [StepEntry(f"s{i}", [toks[-1]], [0]) for i, toks in enumerate(short)]
    entries.insert(3, StepEntry("long", long_prompt[120:], [0, 150, 299]))
    out = runner.step(entries).float().cpu()
    runner.check_status()
    assert runner.stats["two_stream_layers"] == CONFIG["num_hidden_layers"]     # the step took the two-stream path
    rows, r = [], 0
    for e in entries:
        if e.request == "long":
            ref = P.forward_logits(cfg, w, long_prompt)[[120, 270, 419]].cpu()
        else:
            ref = P.forward_logits(cfg, w, short[int(e.request[1:])])[-1:].cpu()
        got = out[r : r + ref.shape[0]]
        r += ref.shape[0]
        torch.testing.assert_close(got, ref, atol=0.03 * float(ref.abs().max()), rtol=0.03)
        rows.append((got.argmax(-1) == ref.argmax(-1)).float())
    assert torch.cat(rows).mean() > 0.8
    cache.assert_invariants()


def test_7b_layer_sizes_one_request_far_into_a_long_context(folder, tmp_path):
    """One request 9,000 tokens into its context, bfloat16: a decode step then cuts its keys into several
    clusters per KV head (four KV heads alone would keep 64 CTAs busy), each cluster leaves a part and
    attention_combine merges them.  Twelve tokens decoded one by one through the captured graph are
    compared with the same twelve positions run as the end of a prompt portion by the tcgen05 kernel:
    two paths of the engine over the same cache content (the fixture's weights make attention far from
    uniform)."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    long_folder = tmp_path / "long"
    long_folder.mkdir()
    (long_folder / "config.json").write_text(json.dumps(dict(CONFIG, max_position_embeddings=12000)))
    (long_folder / "model.safetensors").symlink_to(folder / "model.safetensors")
    model = load_model(long_folder, dtype="bfloat16")
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=1200, page_size=16, max_requests=2,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    cluster, groups = runner.batch.slots[0].planner.decode_fixed(1, 16384)
    assert groups > 1 and cluster * groups >= 32
    N, tail = 9000, 12
    tokens = random_tokens(CONFIG["vocab_size"], N + tail, seed=21)
    cache.open("decoded")
    for a in range(0, N, 3000):
        runner.step([StepEntry("decoded", tokens[a:a + 3000], [])])
    one_by_one = [runner.step([StepEntry("decoded", [t], [0])]).float().cpu().clone() for t in tokens[N:]]
    runner.check_status()
    assert runner.stats["graph_steps"] == tail
    cache.open("portion")
    for a in range(0, 8000, 4000):
        runner.step([StepEntry("portion", tokens[a:a + 4000], [])])
    whole = runner.step([StepEntry("portion", tokens[8000:], list(range(1000, 1000 + tail)))]).float().cpu()
    runner.check_status()
    got = torch.cat(one_by_one)
    scale = float(whole.abs().max())
    assert float((got - whole).abs().max()) < 0.02 * scale, float((got - whole).abs().max()) / scale
    assert (got.argmax(-1) == whole.argmax(-1)).float().mean() >= 0.9
    cache.assert_invariants()


def test_7b_layer_sizes_forty_requests_of_uneven_length_decode_together(folder):
    """Forty requests with 20 to 900 cached tokens decode one token each in one captured step, bfloat16:
    one CTA per token and KV head would wait for the longest history, so the planner cuts every token's
    keys into a few shares (more clusters than are resident at once); every row is compared with the
    plain implementation of its own request."""
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    torch.backends.cuda.matmul.allow_tf32 = False
    cfg, w = P.load_folder(folder, dtype=torch.float32, device="cuda:0")
    model = load_model(folder, dtype="bfloat16")
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=1400, page_size=16, max_requests=40,
                                                        dtype=model.rt.dtype))
    runner = ModelRunner(model, cache)
    g = torch.Generator().manual_seed(4)
    lengths = torch.randint(20, 500, (40,), generator=g).tolist()
    lengths[3], lengths[17], lengths[31] = 900, 860, 777
    prompts = [random_tokens(CONFIG["vocab_size"], n, seed=100 + i) for i, n in enumerate(lengths)]
    for i, toks in enumerate(prompts):
        cache.open(f"r{i}")
    for a in range(0, 40, 8):                                 # prefill all but the last token, eight requests a step
        runner.step([StepEntry(f"r{i}", prompts[i][:-1], []) for i in range(a, a + 8)])
    planner = runner.batch.slots[0].planner
    shares = planner.decode_fixed_for(np.asarray([n - 1 for n in lengths]), 1024)
    assert planner.decode_fixed(40, 1024) == (1, 1) and shares[0] > 1
    out = runner.step([StepEntry(f"r{i}", [prompts[i][-1]], [0]) for i in range(40)]).float().cpu()
    runner.check_status()
    assert runner.stats["graph_steps"] == 1
    agree = []
    for i, toks in enumerate(prompts):
        ref = P.forward_logits(cfg, w, toks)[-1].cpu()
        torch.testing.assert_close(out[i], ref, atol=0.03 * float(ref.abs().max()), rtol=0.03)
        agree.append(float(out[i].argmax() == ref.argmax()))
    assert sum(agree) / len(agree) > 0.8
    cache.assert_invariants()
