"""Generality of the parts interface, shown with toy parts defined here and registered
without any change to the package's files: a mixer with per-request state of its own, a
feed-forward with routing, a rotary position encoding, a model whose layers differ (full
attention with grouped heads, a window, the state mixer), a run order in which one layer
reads another layer's cache and one layer runs twice, and a layer of another shape than
the shipped block knows: one norm shared by two mixers side by side (attention fed from three
file tensors, and the state mixer under a cache key of its own), a third norm after them, and
the shared norm again before the feed-forward.  None of this is any published model; the plain float64 reference of the toy model is written out below.
"""
from dataclasses import dataclass
from typing import ClassVar

import numpy as np
import pytest
import torch

import plain_gpt2 as P

pytestmark = pytest.mark.gpu


# ---- toy parts (torch ops; the framework only sees the interfaces) ----------------------------

def register_toys():
    from rosellm_b200.config.base import ModelConfig, register_architecture, require
    from rosellm_b200.parts import (Concat, LayerSpec, ModelSpec, ParamSpec, Part, PartSpec, RunEntry, StateSpec,
                                    register_part)

    @register_part("mixer", "toy_decaying_sum")
    class DecayingSum(Part):
        """s_t = decay * s_{t-1} + h_t per request, carried across steps in a state slot;
        x += s_t W^T."""

        def __init__(self, hidden_size: int, decay: float):
            self.hidden_size, self.decay = hidden_size, decay
            self.weight = None

        def param_specs(self):
            return [ParamSpec("weight", (self.hidden_size, self.hidden_size))]

        def state_spec(self):
            return StateSpec((self.hidden_size,), torch.float32)

        def forward(self, ctx, run, h, x):
            state = ctx.state(run.state_key)
            qs = ctx.host.q_start
            for r, slot in enumerate(ctx.host.slots.tolist()):
                s = state[slot].clone()
                for t in range(int(qs[r]), int(qs[r + 1])):
                    s = self.decay * s + h[t].float()
                    x[t] += s @ self.weight.float().t()
                state[slot] = s

    @register_part("feed_forward", "toy_routed")
    class Routed(Part):
        """Two experts, each a square matrix; a token goes to the expert whose router row
        scores it higher (router in float32)."""

        def __init__(self, hidden_size: int):
            self.hidden_size = hidden_size
            self.router = self.expert0 = self.expert1 = None

        def param_specs(self):
            d = self.hidden_size
            return [ParamSpec("router", (2, d), kind="vector"), ParamSpec("expert0", (d, d)), ParamSpec("expert1", (d, d))]

        def forward(self, ctx, h, x):
            hf = h.float()
            pick = (hf @ self.router.t()).argmax(-1)
            y0, y1 = hf @ self.expert0.float().t(), hf @ self.expert1.float().t()
            x += torch.where(pick[:, None] == 0, y0, y1)

    @register_part("position", "toy_rotary")
    class Rotary(Part):
        """Pairs (2i, 2i+1) of every head of q and k turned by position * base^(-2i/head_dim)."""

        def __init__(self, head_dim: int, base: float):
            self.head_dim, self.base = head_dim, base

        def table(self):
            return None

        def rotate(self, ctx, q, k):
            half = self.head_dim // 2
            freq = self.base ** (-torch.arange(half, device=q.device, dtype=torch.float32) * 2 / self.head_dim)
            ang = ctx.positions.float()[:, None] * freq[None, :]
            cos, sin = ang.cos()[:, None, :], ang.sin()[:, None, :]
            for t in (q, k):
                v = t.reshape(t.shape[0], -1, half, 2).float()
                a, b = v[..., 0], v[..., 1]
                out = torch.stack([a * cos - b * sin, a * sin + b * cos], dim=-1)
                t.copy_(out.reshape(t.shape[0], -1).to(t.dtype))

    @register_part("block", "toy_two_branches")
    class TwoBranches(Part):
        """``y = mixer(n(x)) + mixer_b(n(x)); x += post_norm(y); x += feed_forward(n(x))`` with one
        norm ``n`` used twice: five sub-parts under names of this block's own choosing."""

        uses = {"norm_shared": "norm", "mixer": "mixer", "mixer_b": "mixer", "post_norm": "norm",
                "feed_forward": "feed_forward"}

        def forward(self, ctx, run, layer, x):
            h = layer.norm_shared.forward(ctx, x, name="toy_shared")
            y = torch.zeros_like(x)
            layer.mixer.forward(ctx, run, h, y)
            layer.mixer_b.forward(ctx, run.for_part("mixer_b"), h, y)
            x += layer.post_norm.forward(ctx, y, name="toy_post").float()
            h = layer.norm_shared.forward(ctx, x, name="toy_shared")
            layer.feed_forward.forward(ctx, h, x)

    @dataclass(frozen=True)
    class ToyConfig(ModelConfig):
        architecture: ClassVar[str] = "ToyMixedLM"
        width: int
        words: int
        longest: int
        decay: float
        window: int
        eps: float
        base: float

        @classmethod
        def from_dict(cls, raw):
            return cls(require(raw, "width", int), require(raw, "words", int), require(raw, "longest", int),
                       require(raw, "decay", float), require(raw, "window", int), require(raw, "eps", float),
                       require(raw, "base", float))

        def to_dict(self):
            return {"architectures": [self.architecture], **self.flat()}

    def build(c):
        d = c.width

        def norm(name):
            return PartSpec("layer_norm", dict(hidden_size=d, eps=c.eps), {"weight": name + ".g", "bias": name + ".b"})

        def attn(i, window):
            return PartSpec("causal_self_attention",
                            dict(hidden_size=d, num_heads=4, head_dim=16, num_kv_heads=2, window=window, bias=False),
                            {"qkv_weight": f"l{i}.qkv", "out_weight": f"l{i}.o"})

        def mlp(i):
            return PartSpec("dense_mlp", dict(hidden_size=d, inner_size=3 * d, activation="gelu_erf", bias=False),
                            {"in_weight": f"l{i}.up", "out_weight": f"l{i}.down"})

        def layer(i, mixer, ff):
            return LayerSpec.standard(PartSpec("pre_norm"), mixer, ff, norm(f"l{i}.n1"), norm(f"l{i}.n2"))

        layers = (
            layer(0, attn(0, None), mlp(0)),
            layer(1, PartSpec("toy_decaying_sum", dict(hidden_size=d, decay=c.decay), {"weight": "l1.mix"}),
                  PartSpec("toy_routed", dict(hidden_size=d), {"router": "l1.router", "expert0": "l1.e0", "expert1": "l1.e1"})),
            layer(2, attn(2, c.window), mlp(2)),
            layer(3, attn(3, None), mlp(3)),
            LayerSpec.of(
                PartSpec("toy_two_branches"),
                norm_shared=("norm", norm("l4.n")),
                # the packed qkv matrix [128, d] from three tensors of the file
                mixer=("mixer", PartSpec("causal_self_attention",
                                         dict(hidden_size=d, num_heads=4, head_dim=16, num_kv_heads=2, bias=False),
                                         {"qkv_weight": Concat(("l4.q", "l4.k", "l4.v"), dim=0, sizes=(64, 32, 32)),
                                          "out_weight": "l4.o"})),
                mixer_b=("mixer", PartSpec("toy_decaying_sum", dict(hidden_size=d, decay=c.decay / 2), {"weight": "l4.mix"})),
                post_norm=("norm", norm("l4.post")),
                feed_forward=("feed_forward", mlp(4)),
            ),
        )
        return ModelSpec(
            hidden_size=d, vocab_size=c.words, max_positions=c.longest,
            embedding=PartSpec("token_table", dict(vocab_size=c.words, hidden_size=d), {"weight": "emb"}),
            position=PartSpec("toy_rotary", dict(head_dim=16, base=c.base)),
            layers=layers,
            # layer 3 reads layer 0's cache; layer 0 then runs a second time over its own cache
            run_order=(RunEntry(0), RunEntry(1), RunEntry(2), RunEntry(3, cache_of=0), RunEntry(0, cache_of=0),
                       RunEntry(4)),
            final_norm=norm("nf"),
            head=PartSpec("linear", dict(vocab_size=c.words, hidden_size=d), {"weight": "head"}),
        )

    register_architecture("ToyMixedLM", ToyConfig, build, replace=True)
    return ToyConfig


def unregister_toys():
    from rosellm_b200.config.base import unregister_architecture
    from rosellm_b200.parts import unregister_part

    unregister_architecture("ToyMixedLM")
    for cat, kind in (("mixer", "toy_decaying_sum"), ("feed_forward", "toy_routed"), ("position", "toy_rotary"),
                      ("block", "toy_two_branches")):
        unregister_part(cat, kind)


# ---- the toy model written out plainly (float64, whole sequence, no cache) -----------------------

def plain_toy(c, t, ids):
    T, d = len(ids), c.width
    t = {k: v.double() for k, v in t.items()}
    x = t["emb"][torch.tensor(ids)]
    pos = torch.arange(T, dtype=torch.float64)
    freq = c.base ** (-torch.arange(8, dtype=torch.float64) * 2 / 16)
    cos, sin = (pos[:, None] * freq).cos()[:, None, :], (pos[:, None] * freq).sin()[:, None, :]

    def rot(v):  # [T, heads, 16]
        a, b = v[..., 0::2], v[..., 1::2]
        return torch.stack([a * cos - b * sin, a * sin + b * cos], -1).reshape(v.shape)

    def ln(x, name):
        return P.layer_norm(x, t[name + ".g"], t[name + ".b"], c.eps)

    def attend(q, k, v, window):
        k, v = k.repeat_interleave(2, 1), v.repeat_interleave(2, 1)
        s = torch.einsum("thd,shd->hts", q, k) * 16 ** -0.5
        i = torch.arange(T)
        vis = i[None, :] <= i[:, None]
        if window is not None:
            vis &= i[None, :] > i[:, None] - window
        return torch.einsum("hts,shd->thd", torch.softmax(s.masked_fill(~vis, float("-inf")), -1), v).reshape(T, 64)

    def qkv(i, h):
        q, k, v = (h @ t[f"l{i}.qkv"].t()).split([64, 32, 32], -1)
        return rot(q.view(T, 4, 16)), rot(k.view(T, 2, 16)), v.view(T, 2, 16)

    def mlp(i, h):
        return P.gelu_erf(h @ t[f"l{i}.up"].t()) @ t[f"l{i}.down"].t()

    # layer 0
    q0, k0, v0 = qkv(0, ln(x, "l0.n1"))
    x = x + attend(q0, k0, v0, None) @ t["l0.o"].t()
    x = x + mlp(0, ln(x, "l0.n2"))
    # layer 1: decaying sum, routed feed-forward
    h = ln(x, "l1.n1")
    s = torch.zeros(d, dtype=torch.float64)
    ys = []
    for i in range(T):
        s = c.decay * s + h[i]
        ys.append(s @ t["l1.mix"].t())
    x = x + torch.stack(ys)
    h = ln(x, "l1.n2")
    scores = h @ t["l1.router"].t()
    pick = scores.argmax(-1)
    margin = float((scores[:, 0] - scores[:, 1]).abs().min())
    x = x + torch.where(pick[:, None] == 0, h @ t["l1.e0"].t(), h @ t["l1.e1"].t())
    # layer 2: window
    q, k, v = qkv(2, ln(x, "l2.n1"))
    x = x + attend(q, k, v, c.window) @ t["l2.o"].t()
    x = x + mlp(2, ln(x, "l2.n2"))
    # layer 3 over layer 0's keys and values
    q, _, _ = qkv(3, ln(x, "l3.n1"))
    x = x + attend(q, k0, v0, None) @ t["l3.o"].t()
    x = x + mlp(3, ln(x, "l3.n2"))
    # layer 0 again, over the cache its first run left
    q, _, _ = qkv(0, ln(x, "l0.n1"))
    x = x + attend(q, k0, v0, None) @ t["l0.o"].t()
    x = x + mlp(0, ln(x, "l0.n2"))
    # layer 4: one norm for two mixers side by side, a norm after them, the first norm again
    h = ln(x, "l4.n")
    q = rot((h @ t["l4.q"].t()).view(T, 4, 16))
    k = rot((h @ t["l4.k"].t()).view(T, 2, 16))
    v = (h @ t["l4.v"].t()).view(T, 2, 16)
    y = attend(q, k, v, None) @ t["l4.o"].t()
    s = torch.zeros(d, dtype=torch.float64)
    ys = []
    for i in range(T):
        s = c.decay / 2 * s + h[i]
        ys.append(s @ t["l4.mix"].t())
    x = x + ln(y + torch.stack(ys), "l4.post")
    x = x + mlp(4, ln(x, "l4.n"))
    return ln(x, "nf") @ t["head"].t(), margin


@pytest.fixture
def toy(tmp_path):
    ToyConfig = register_toys()
    try:
        from rosellm_b200.weights import read_safetensors, write_model_folder

        cfg = ToyConfig(width=64, words=90, longest=96, decay=0.8, window=7, eps=1e-4, base=100.0)
        folder = write_model_folder(cfg, 11, str(tmp_path / "toy"), std=0.25)
        yield cfg, folder, read_safetensors(folder)
    finally:
        unregister_toys()


@pytest.mark.parametrize("dtype,atol", [("float32", 2e-4), ("bfloat16", 0.35)])
def test_toy_model_is_registered_built_and_stepped(toy, dtype, atol):
    from rosellm_b200.config import EngineConfig
    from rosellm_b200.engine.runner import ModelRunner, StepEntry

    cfg, folder, tensors = toy
    runner = ModelRunner.from_folder(folder, EngineConfig(dtype=dtype, page_size=4, kv_cache_tokens=256,
                                                          max_num_seqs=4, max_num_batched_tokens=128))
    assert not runner.model.graph_safe  # the toy parts read index arrays on the host
    cache = runner.cache
    assert sorted(g.spec.window for g in cache.groups if g.spec.window) == [7] and len(cache.groups) == 2
    assert list(cache.states) == [1, (4, "mixer_b")] and cache.state(1).shape == (4, 64)
    assert cache.state((4, "mixer_b")).shape == (4, 64) and 4 in cache.group_of_layer
    # Routing is a discontinuity: a token whose two router scores nearly tie may go to the
    # other expert under bfloat16 rounding, which is no fault.  Take the first token
    # sequences whose smallest margin is well clear of that rounding.
    for seed in range(200):
        rng = np.random.default_rng(seed)
        seqs = {"a": rng.integers(0, 90, 50).tolist(), "b": rng.integers(0, 90, 23).tolist(),
                "c": rng.integers(0, 90, 9).tolist()}
        plain = {k: plain_toy(cfg, tensors, v) for k, v in seqs.items()}
        if min(m for _, m in plain.values()) > 0.15:
            break
    else:
        raise AssertionError("no token sequences with a clear routing margin")
    want = {k: v[0] for k, v in plain.items()}
    slots = {k: cache.new_request() for k in ("a", "b")}
    at = {k: 0 for k in seqs}
    worst = 0.0

    def step(parts):
        nonlocal worst
        entries = [StepEntry(slots[k], seqs[k][at[k]:at[k] + n], list(range(n))) for k, n in parts]
        logits = runner.step(entries).double().cpu()
        runner.check_status()
        row = 0
        for k, n in parts:
            diff = float((logits[row:row + n] - want[k][at[k]:at[k] + n]).abs().max())
            assert diff <= atol, f"request {k} tokens {at[k]}..{at[k] + n}: {diff:.3e}"
            worst = max(worst, diff)
            row += n
            at[k] += n

    step([("a", 13), ("b", 2)])
    step([("a", 1), ("b", 9)])
    step([("a", 1)])                       # b sits this step out
    step([("a", 20), ("b", 1)])
    step([("b", 11), ("a", 2)])
    assert at["b"] == 23
    cache.release(slots.pop("b"))          # c takes b's slot, pages and state row
    slots["c"] = cache.new_request()
    step([("a", 13), ("c", 5)])
    step([("c", 1)])
    step([("c", 3)])
    assert at == {"a": 50, "b": 23, "c": 9}
    win = next(i for i, g in enumerate(cache.groups) if g.spec.window)
    assert len(cache.pages_of(slots["a"], win)) <= 3 < len(cache.pages_of(slots["a"], 1 - win))
    for s in slots.values():
        cache.release(s)
    cache.check()
    assert all(g.allocator.num_free == cache.num_pages for g in cache.groups)
