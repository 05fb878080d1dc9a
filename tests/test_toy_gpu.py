"""Generality of the parts: a toy model defined HERE, with a mixer that keeps a state of its own,
a feed-forward that routes each token to one of two experts, a position encoding of its own
(rotary with stretched wavelengths), a layer that runs twice, a layer that reads another layer's
cache, a layer without position encoding, a layer whose attention has twice the query heads over
the same keys (it shares the other layers' pages and block table) with interleaved rotation of
half of each head, and a block arrangement of its own with one norm more than the built-in one,
is registered, built from a model folder and stepped in portions, without a change to the
framework's files.  It is compared with a whole-sequence computation written here.  None of
these toys is anyone's model."""
import json
from dataclasses import dataclass

import pytest
import torch

from conftest import random_tokens
from plain import qwen2_plain as P

pytestmark = pytest.mark.gpu

TOY = dict(architectures=["ToyForCausalLM"], vocab_size=130, hidden_size=48, intermediate_size=72,
           q_heads=3, kv_heads=1, head_dim=16, eps=1e-5, theta=777.0)


def register_toy():
    from mini_hisparse_b200 import register_architecture
    from mini_hisparse_b200.parts import (FEED_FORWARDS, MIXERS, NORMS, Block, FeedForward, LayerSpec, Mixer,
                                          ModelSpec, ParamSpec, PartSpec, Product, RunEntry, StateNeed,
                                          register_block, register_feed_forward, register_mixer,
                                          register_position)
    from mini_hisparse_b200.parts.position import Position

    @register_position("toy_stretched_rotary", replace=True)
    class StretchedRotary(Position):
        """Half-split rotation whose wavelengths are `stretch` times longer."""

        def __init__(self, spec, rt=None):
            super().__init__(spec, rt)
            d = spec["head_dim"]
            self.rotary_dim = d
            inv = spec["theta"] ** (-torch.arange(0, d, 2).float() / d) / spec["stretch"]
            self.inv_freq = inv.to(rt.device) if rt is not None else inv

    @register_block("toy_sandwich", replace=True)
    class SandwichBlock(Block):
        """x = x + post_norm(mixer(norm(x))); x = x + ff(norm2(x)): the built-in arrangement with a
        fifth part, a norm on the mixer's output."""

        graph_safe = False          # reduced() below is plain torch: a toy

        def __init__(self, spec, rt):
            self.spec = spec
            self.mixer_norm = NORMS.build(spec.part("mixer_norm"), rt=rt)
            self.mixer = MIXERS.build(spec.part("mixer"), rt=rt)
            self.post_norm = NORMS.build(spec.part("post_norm"), rt=rt)
            self.ff_norm = NORMS.build(spec.part("ff_norm"), rt=rt)
            self.feed_forward = FEED_FORWARDS.build(spec.part("feed_forward"), rt=rt)

        def parts(self):
            return {"mixer_norm": self.mixer_norm, "mixer": self.mixer, "post_norm": self.post_norm,
                    "ff_norm": self.ff_norm, "feed_forward": self.feed_forward}

        def forward(self, x, pending, ctx, cache):
            h = self.mixer_norm.forward(x, ctx, delta=pending)
            a = self.mixer.forward(h, ctx, cache).reduced().contiguous()     # float32 [T, H]
            post = self.post_norm.forward(a, ctx, name="toy_post")
            h = self.ff_norm.forward(x, ctx, delta=Product(post))
            return self.feed_forward.forward(h, ctx)

    @register_feed_forward("toy_routed", replace=True)
    class Routed(FeedForward):
        """Each token goes to the expert with the larger router logit (float32); an expert is
        a two-matrix ReLU network.  Plain torch on the device: a toy, not a product path."""

        graph_safe = False

        def __init__(self, spec, rt=None):
            super().__init__(spec, rt)
            self.h, self.i = spec["hidden_size"], spec["intermediate_size"]

        def parameters(self):
            p = {"router.weight": ParamSpec((2, self.h))}
            for e in range(2):
                p[f"experts.{e}.w1.weight"] = ParamSpec((self.i, self.h))
                p[f"experts.{e}.w2.weight"] = ParamSpec((self.h, self.i))
            return p

        def load(self, tensors):
            self.t = {k: v.float() for k, v in tensors.items()}

        def forward(self, h, ctx):
            x = h.float()
            choice = (x @ self.t["router.weight"].T).argmax(-1)
            out = torch.zeros_like(x)
            for e in range(2):
                rows = choice == e
                out[rows] = torch.relu(x[rows] @ self.t[f"experts.{e}.w1.weight"].T) @ self.t[f"experts.{e}.w2.weight"].T
            res = ctx.ws.get("toy_ff", tuple(h.shape), ctx.rt.dtype)
            res.copy_(out)
            return Product(res)

    @register_mixer("toy_running_mean", replace=True)
    class RunningMean(Mixer):
        """out[t] = W . mean(h[0..t]); the state is the running sum, carried across steps."""

        graph_safe = False

        def __init__(self, spec, rt=None):
            super().__init__(spec, rt)
            self.width = spec["hidden_size"]

        def cache_need(self):
            return StateNeed(shape=(self.width,), dtype="float32")

        def parameters(self):
            return {"mix.weight": ParamSpec((self.width, self.width))}

        def load(self, tensors):
            self.w = tensors["mix.weight"]

        def forward(self, h, ctx, cache):
            out = ctx.ws.get("toy_out", (h.shape[0], self.width), ctx.rt.dtype)
            for seg in ctx.segments:
                rows = slice(seg.offset, seg.offset + seg.count)
                csum = h[rows].float().cumsum(0) + cache.storage[seg.slot]
                counts = torch.arange(seg.start + 1, seg.start + seg.count + 1, device=h.device)
                if cache.writable:
                    cache.storage[seg.slot] = csum[-1]
                out[rows] = ((csum / counts[:, None]) @ self.w.float().T).to(out.dtype)
            return Product(out)

    @dataclass(frozen=True)
    class ToyConfig:
        raw: tuple

        @classmethod
        def from_dict(cls, d):
            return cls(tuple(sorted((k, v) for k, v in d.items() if k != "architectures")))

        def __getitem__(self, k):
            return dict(self.raw)[k]

    def toy_spec(c):
        H = c["hidden_size"]
        norm = PartSpec.make("rmsnorm", width=H, eps=c["eps"])
        ff = PartSpec.make("swiglu", hidden_size=H, intermediate_size=c["intermediate_size"])

        def attn(position, q_heads=c["q_heads"]):
            return PartSpec.make("gq_attention", hidden_size=H, q_heads=q_heads, kv_heads=c["kv_heads"],
                                 head_dim=c["head_dim"], qkv_bias=False, window=None, position=position)

        rotary = PartSpec.make("toy_stretched_rotary", head_dim=c["head_dim"], theta=c["theta"], stretch=4.0)
        pairs = PartSpec.make("rotary", head_dim=c["head_dim"], theta=c["theta"], style="interleaved",
                              rotary_dim=c["head_dim"] // 2)
        routed = PartSpec.make("toy_routed", hidden_size=H, intermediate_size=c["intermediate_size"])
        mixers = [attn(rotary), PartSpec.make("toy_running_mean", hidden_size=H), attn(PartSpec.make("none"))]
        ffs = [ff, routed, ff]
        layers = [LayerSpec.pre_norm(f"toy.layers.{i}", mixer=m, mixer_norm=norm, feed_forward=f, ff_norm=norm)
                  for i, (m, f) in enumerate(zip(mixers, ffs))]
        # a fourth layer in an arrangement of its own: five parts, twice the query heads, other rotation
        layers.append(LayerSpec.make("toy.layers.3", "toy_sandwich",
                                     {"mixer_norm": norm, "mixer": attn(pairs, 2 * c["q_heads"]), "post_norm": norm,
                                      "ff_norm": norm, "feed_forward": ff},
                                     {"mixer": "self_attn", "feed_forward": "mlp"}))
        layers = tuple(layers)
        order = (RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(1), RunEntry(2, cache_of=2), RunEntry(3))
        return ModelSpec("ToyForCausalLM", c["vocab_size"], H,
                         PartSpec.make("token_embedding", vocab_size=c["vocab_size"], hidden_size=H), "toy.embed",
                         layers, order, norm, "toy.norm",
                         PartSpec.make("lm_head", vocab_size=c["vocab_size"], hidden_size=H, tied=True), "toy.head")

    register_architecture("ToyForCausalLM", ToyConfig, toy_spec, replace=True)


def toy_reference(w, tokens):
    """The whole sequence at once, from the formulas above."""
    c = TOY
    T = len(tokens)
    x = w["toy.embed.weight"][torch.tensor(tokens)]
    pos = torch.arange(T)
    shared_kv = {}

    def interleaved_half(t):
        """Pairs (2i, 2i + 1) of the first half of every head turned by pos * theta^(-2i / (d/2))."""
        r = c["head_dim"] // 2
        inv = c["theta"] ** (-torch.arange(0, r, 2).float() / r)
        ang = pos.float()[:, None] * inv[None, :]
        cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
        out = t.clone()
        a, b = t[..., 0:r:2], t[..., 1:r:2]
        out[..., 0:r:2], out[..., 1:r:2] = a * cos - b * sin, b * cos + a * sin
        return out

    def attention(i, h, rotate, entry, reuse=None, q_heads=c["q_heads"]):
        p = f"toy.layers.{i}.self_attn."
        q = (h @ w[p + "q_proj.weight"].T).view(T, q_heads, c["head_dim"])
        k = (h @ w[p + "k_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
        v = (h @ w[p + "v_proj.weight"].T).view(T, c["kv_heads"], c["head_dim"])
        if rotate == "interleaved_half":
            q, k = interleaved_half(q), interleaved_half(k)
        elif rotate:
            inv = c["theta"] ** (-torch.arange(0, c["head_dim"], 2).float() / c["head_dim"]) / 4.0
            ang = pos.float()[:, None] * inv[None, :]
            ang = torch.cat((ang, ang), -1)[:, None, :]
            q, k = P.rotate(q, ang.cos(), ang.sin()), P.rotate(k, ang.cos(), ang.sin())
        if reuse is not None:
            k, v = shared_kv[reuse]
        shared_kv[entry] = (k, v)
        return P.causal_attention(q, k, v).reshape(T, -1) @ w[p + "o_proj.weight"].T

    def running_mean(i, h):
        mean = h.cumsum(0) / torch.arange(1, T + 1)[:, None]
        return mean @ w[f"toy.layers.{i}.self_attn.mix.weight"].T

    def routed(i, h):
        p = f"toy.layers.{i}.mlp."
        choice = (h @ w[p + "router.weight"].T).argmax(-1)
        out = torch.zeros_like(h)
        for e in range(2):
            rows = choice == e
            out[rows] = torch.relu(h[rows] @ w[p + f"experts.{e}.w1.weight"].T) @ w[p + f"experts.{e}.w2.weight"].T
        return out

    def block(i, x, mix):
        p = f"toy.layers.{i}."
        x = x + mix(P.rms_norm(x, w[p + "input_layernorm.weight"], c["eps"]))
        h = P.rms_norm(x, w[p + "post_attention_layernorm.weight"], c["eps"])
        if i == 1:
            return x + routed(i, h)
        return x + P.swiglu(h, w[p + "mlp.gate_proj.weight"], w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])

    x = block(0, x, lambda h: attention(0, h, True, 0))
    x = block(1, x, lambda h: running_mean(1, h))
    x = block(2, x, lambda h: attention(2, h, False, 2))
    x = block(1, x, lambda h: running_mean(1, h))
    x = block(2, x, lambda h: attention(2, h, False, 4, reuse=2))
    # the sandwich arrangement: a norm on the mixer's output before it joins the residual
    p = "toy.layers.3."
    a = attention(3, P.rms_norm(x, w[p + "mixer_norm.weight"], c["eps"]), "interleaved_half", 5,
                  q_heads=2 * c["q_heads"])
    x = x + P.rms_norm(a, w[p + "post_norm.weight"], c["eps"])
    x = x + P.swiglu(P.rms_norm(x, w[p + "ff_norm.weight"], c["eps"]), w[p + "mlp.gate_proj.weight"],
                     w[p + "mlp.up_proj.weight"], w[p + "mlp.down_proj.weight"])
    return P.rms_norm(x, w["toy.norm.weight"], c["eps"]) @ w["toy.embed.weight"].T


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_toy_model_registers_builds_and_steps(tmp_path, dtype):
    from mini_hisparse_b200 import CacheConfig, CacheManager, load_model, write_random_model
    from mini_hisparse_b200.engine import ModelRunner, StepEntry

    register_toy()
    write_random_model(TOY, 5, tmp_path, dtype=torch.bfloat16, matrix_std=0.15)
    w = {k: v.float() for k, v in P.read_safetensors(tmp_path / "model.safetensors").items()}
    model = load_model(tmp_path, dtype=dtype)
    assert len(model.cache_needs) == 5            # six run entries, one of them reads another's cache
    cache = CacheManager(model.cache_needs, CacheConfig(num_pages=12, page_size=16, max_requests=3,
                                                        dtype=model.rt.dtype))
    # the layer with twice the query heads keeps the same keys and values: one pool, one block table
    assert len(cache.page_groups) == 1 and len(cache.state_groups) == 1
    assert len(cache.page_groups[0].entries) == 3 and len(cache.state_groups[0].entries) == 2
    runner = ModelRunner(model, cache)
    assert len(runner.batch.slots) == 2           # ... but a plan of its own
    assert not runner.use_graphs                  # the toy mixer works on the host: no captured graph
    reqs = {"a": random_tokens(130, 70, 1), "b": random_tokens(130, 41, 2)}
    refs = {k: toy_reference(w, t) for k, t in reqs.items()}
    got = {k: [] for k in reqs}
    done = {k: 0 for k in reqs}
    cuts = {"a": [30, 2, 1, 17, 1, 19], "b": [5, 1, 1, 30, 2, 2]}
    for k in reqs:
        cache.open(k)
    for step in range(6):
        entries = []
        for k in reqs:
            n = cuts[k][step]
            entries.append(StepEntry(k, reqs[k][done[k]: done[k] + n], list(range(n))))
        logits = runner.step(entries).cpu()
        runner.check_status()
        row = 0
        for e in entries:
            n = len(e.tokens)
            got[e.request].append(logits[row: row + n].clone())
            row += n
            done[e.request] += n
    for k in reqs:
        out = torch.cat(got[k])
        tol = dict(atol=3e-5, rtol=3e-5) if dtype == "float32" else dict(atol=0.03 * float(refs[k].abs().max()), rtol=0.03)
        torch.testing.assert_close(out, refs[k], **tol)
    # a slot that is used again starts from a zero state
    cache.close("a")
    cache.open("c")
    logits = runner.step([StepEntry("c", reqs["b"][:9], list(range(9)))]).cpu()
    torch.testing.assert_close(logits, refs["b"][:9], **tol)
    cache.assert_invariants()
